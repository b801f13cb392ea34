"""Inter-stage transfer of activations and gradients.

The reference moves one tensor per micro-batch per stage boundary with blocking
``torch.distributed`` send/recv over NCCL (``deepspeed/runtime/pipe/p2p_direct.py:7-17``,
called from ``deepspeed/runtime/pipe/engine.py:1894-2082``) after a three-message shape
handshake (``engine.py:1781-1892``).  Here the engine talks to a ``Transport``:

* ``MailboxTransport`` - the CUDA path.  Every rank owns receive mailboxes (one slot per
  pipeline buffer) that its neighbours map through CUDA IPC; a sender runs a store kernel
  that writes the payload straight into the neighbour's slot over NVLink and then releases
  a sequence flag; the receiver runs a bounded-wait kernel on its own memory and copies
  the slot out.  No NCCL send/recv, no shape handshake (the slot header carries shape and
  dtype), no unbounded spin: a wait that runs out reports ``BB_STATUS_PEER_TIMEOUT`` and
  the engine turns that into its next/previous-stage failure handling.
* ``DistTransport`` - ``torch.distributed`` isend/recv; used for the CPU (gloo) plumbing
  configuration and the host-logic tests.  It refuses CUDA tensors.
* ``NullTransport`` - single-stage pipelines.
"""
import time
from datetime import timedelta
from typing import Dict, Optional, Tuple

import torch

ACT, GRAD, PING = 0, 1, 2


class PeerTimeout(RuntimeError):
    """The neighbour did not produce / accept a message within the time limit."""

    def __init__(self, peer, msg=""):
        super().__init__(msg or f"peer rank {peer} timed out")
        self.peer = peer


class NullTransport:
    name = "null"

    def send(self, tensor, dst, kind, slot, seq):
        raise RuntimeError("single-stage pipeline has no neighbours")

    def recv(self, src, kind, slot, seq):
        raise RuntimeError("single-stage pipeline has no neighbours")

    send_ping = send
    recv_ping = recv

    def exchange_state(self, send_to, tensors_out, recv_from, tensors_in, seq):
        return

    def end_step(self):
        return

    def close(self):
        return


_DTYPES = [torch.float32, torch.bfloat16, torch.float16, torch.int64, torch.int32, torch.uint8, torch.float64]


class DistTransport:
    """torch.distributed point-to-point (gloo on CPU).  Sends are asynchronous and are
    completed at ``end_step``; receives block with a timeout."""

    name = "dist"

    def __init__(self, dist, timeout_s=30.0):
        self.dist = dist
        self.timeout_s = timeout_s
        self._pending = []
        self._meta: Dict[Tuple[int, int], Tuple[torch.Size, torch.dtype]] = {}
        self._sent_meta = set()
        # establish every pairwise connection up front (the reference "sends a 0" between
        # neighbours at engine start for the same reason, pipe/engine.py:259-269)
        dist.barrier()

    @staticmethod
    def _check_cpu(t):
        if t.is_cuda:
            raise RuntimeError("DistTransport is the CPU plumbing path; CUDA stages use MailboxTransport "
                               "(no NCCL send/recv on the activation path)")

    def _wait(self, work, peer):
        # gloo point-to-point work only progresses inside wait(); a timeout surfaces as an error
        try:
            work.wait(timedelta(seconds=self.timeout_s))
        except RuntimeError as e:
            raise PeerTimeout(peer, f"peer rank {peer}: {str(e)[:200]}")

    def send(self, tensor, dst, kind, slot, seq):
        self._check_cpu(tensor)
        t = tensor.detach().contiguous()
        try:
            if (dst, kind) not in self._sent_meta:
                meta = torch.zeros(10, dtype=torch.int64)
                meta[0], meta[1] = _DTYPES.index(t.dtype), t.dim()
                meta[2:2 + t.dim()] = torch.tensor(list(t.shape), dtype=torch.int64)
                self._pending.append((self.dist.isend(meta, dst, tag=kind), dst, meta))
                self._sent_meta.add((dst, kind))
            self._pending.append((self.dist.isend(t, dst, tag=kind), dst, t))
        except RuntimeError as e:  # the connection to a dead peer is already closed
            raise PeerTimeout(dst, f"peer rank {dst}: {str(e)[:200]}")

    def _irecv(self, buf, src, tag):
        try:
            return self.dist.irecv(buf, src, tag=tag)
        except RuntimeError as e:
            raise PeerTimeout(src, f"peer rank {src}: {str(e)[:200]}")

    def recv(self, src, kind, slot, seq):
        if (src, kind) not in self._meta:
            meta = torch.zeros(10, dtype=torch.int64)
            self._wait(self._irecv(meta, src, kind), src)
            nd = int(meta[1])
            self._meta[(src, kind)] = (torch.Size(meta[2:2 + nd].tolist()), _DTYPES[int(meta[0])])
        shape, dtype = self._meta[(src, kind)]
        buf = torch.empty(shape, dtype=dtype)
        self._wait(self._irecv(buf, src, kind), src)
        return buf

    def send_ping(self, dst, seq):
        t = torch.full((1,), float(seq))
        try:
            self._pending.append((self.dist.isend(t, dst, tag=PING), dst, t))
        except RuntimeError as e:
            raise PeerTimeout(dst, f"peer rank {dst}: {str(e)[:200]}")

    def recv_ping(self, src, seq):
        t = torch.zeros(1)
        self._wait(self._irecv(t, src, PING), src)

    def exchange_state(self, send_to, tensors_out, recv_from, tensors_in, seq):
        """Ship this stage's flat optimizer state to the rank shadowing it and take the
        successor's into the local shadow buffers."""
        works, staged = [], []
        peer = send_to
        try:
            if send_to is not None:
                for t in tensors_out:
                    self._check_cpu(t)
                    works.append((self.dist.isend(t.detach().contiguous(), send_to, tag=3), send_to))
            if recv_from is not None:
                # received into staging buffers and moved over only when every piece is in, so a
                # sender that dies half way leaves the shadow whole (one step old), never torn
                peer = recv_from
                for t in tensors_in:
                    buf = torch.empty_like(t)
                    staged.append((t, buf))
                    works.append((self.dist.irecv(buf, recv_from, tag=3), recv_from))
        except RuntimeError as e:  # connection already closed by a dead peer
            raise PeerTimeout(peer, str(e)[:200])
        send_err = recv_err = None
        n_send = len(works) - len(staged)
        for i, (w, peer) in enumerate(works):
            try:
                self._wait(w, peer)
            except PeerTimeout as e:
                if i < n_send:
                    send_err = send_err or e
                else:
                    recv_err = recv_err or e
        if recv_err is None:
            for t, buf in staged:
                t.copy_(buf)
        if recv_err is not None or send_err is not None:
            raise recv_err or send_err

    def forget_peer(self, peer):
        for k in [k for k in self._meta if k[0] == peer]:
            del self._meta[k]
        self._sent_meta = {k for k in self._sent_meta if k[0] != peer}

    def end_step(self):
        for w, peer, _keep in self._pending:
            try:
                self._wait(w, peer)
            except PeerTimeout:
                pass  # a dead receiver; the failure is handled where a receive needs it
        self._pending = []

    def close(self):
        self._pending = []
