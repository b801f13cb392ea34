"""Data loading helpers of the training step.

``RepeatingLoader`` restarts its iterator on exhaustion.  The reference's version
(``deepspeed/runtime/dataloader.py:10-31``) builds a new iterator on *every* ``__next__``
and therefore returns the first batch forever; this one keeps the iterator, which is what
its docstring promises.  ``build_loader`` follows ``PipelineEngine._build_data_iter``
(``deepspeed/runtime/pipe/engine.py:882-891``): an unshuffled distributed sampler over the
data-parallel replicas, micro-batch sized batches.
"""
import torch


class RepeatingLoader:
    def __init__(self, loader):
        self.loader = loader
        self.data_iter = iter(loader)

    def __iter__(self):
        return self

    def __next__(self):
        try:
            return next(self.data_iter)
        except StopIteration:
            self.data_iter = iter(self.loader)
            return next(self.data_iter)


def build_loader(dataset, micro_batch_size, dp_world_size, dp_rank, collate_fn=None):
    sampler = torch.utils.data.distributed.DistributedSampler(dataset, num_replicas=dp_world_size, rank=dp_rank,
                                                              shuffle=False)
    return torch.utils.data.DataLoader(dataset, batch_size=micro_batch_size, sampler=sampler, collate_fn=collate_fn,
                                       pin_memory=torch.cuda.is_available(), drop_last=True)
