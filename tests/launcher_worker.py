"""Training script started by the node agent in tests/test_launcher.py: everything it knows comes from
the environment the agent gave it."""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    out_dir = os.environ["LAUNCHER_TEST_OUT"]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    node = os.environ.get("LAUNCHER_TEST_NODE", "x")
    attempt_marker = os.path.join(out_dir, f"standby_once_{node}")
    if os.environ.get("LAUNCHER_TEST_STANDBY_ONCE") and not os.path.exists(attempt_marker):
        # what a reconfiguration looks like from the agents' side: the active rendezvous version is withdrawn
        # (the engine's reconfiguration decision does that) and the workers end with 125 - "form the job anew"
        import time
        from bamboo_b200.rendezvous import handler_from_env
        open(attempt_marker, "w").write("1")
        impl = handler_from_env()._rdzv_impl
        key = impl.get_path("/rdzv/active_version")
        if rank == 0:
            impl.client.delete(key)
        else:
            deadline = time.time() + 60
            while time.time() < deadline:
                try:
                    impl.client.get(key)
                    time.sleep(0.05)
                except Exception:
                    break
        sys.exit(125)
    import cpu_layers
    from oracle import gpt_ref
    from bamboo_b200 import api
    from bamboo_b200.module import PipelineModule
    from bamboo_b200.rendezvous import grid_from_env, handler_from_env
    from bamboo_b200.topology import PipeDataParallelTopology
    torch.set_num_threads(1)
    os.environ.setdefault("BAMBOO_QUIET", "1")
    cfg = gpt_ref.RefConfig(layers=2, hidden=32, heads=2, ffn=64, seq=8, vocab=48)
    dist.init_process_group("gloo", rank=rank, world_size=world)          # env:// with the agent's MASTER_ADDR / MASTER_PORT
    num_dp, num_pp, coords = grid_from_env()
    handler = handler_from_env()
    topo = PipeDataParallelTopology(num_pp=num_pp, num_dp=num_dp, custom_mapping=handler.get_global_decision())
    model = PipelineModule(cpu_layers.ref_layer_specs(cfg, 0), topology=topo, loss_fn=cpu_layers.ref_loss(cfg),
                           partition_method="uniform", device="cpu")
    config = {"train_micro_batch_size_per_gpu": 2, "gradient_accumulation_steps": 2,
              "optimizer": {"type": "Adam", "params": {"lr": 1e-3}}, "bamboo_b200": {"p2p_timeout_s": 60}}
    engine, *_ = api.initialize(model=model, config=config, redundancy_level=1, rdzv_handler=handler)
    data = gpt_ref.synthetic_batches(cfg, 2, 2, 2, seed=1)
    losses = [float(engine.train_batch(data_iter=iter(data[s]))) for s in range(2)]
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump({"rank": rank, "stage": engine.stage_id, "coords": coords, "losses": losses,
                   "restart": os.environ["TORCHELASTIC_RESTART_COUNT"], "blocking_wait": os.environ.get("NCCL_BLOCKING_WAIT"),
                   "store": type(engine.global_store).__name__}, f)
    handler.stop_keep_alive()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
