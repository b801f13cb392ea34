"""MailboxTransport: activations, gradients, pings and shadow state over NVLink stores.

Replaces the blocking NCCL ``dist.send/recv`` of the reference
(``deepspeed/runtime/pipe/p2p_direct.py:7-17`` as used by
``deepspeed/runtime/pipe/engine.py:1894-2082``) and its shape handshake
(``engine.py:1781-1892``).

Per (sender, receiver, kind) there is one *channel*: a mailbox in the receiver's HBM with one
slot per pipeline buffer plus a ping flag.  The receiver allocates it when it first needs
the channel and publishes its CUDA-IPC handle through the job's key/value store; the sender
publishes the message geometry (shape, dtype, slots) the same way, so no tensor-meta
messages travel on the data path.  A send is one store kernel into the mapped mailbox that
ends by releasing the message's sequence number into the slot flag; a receive is one kernel
that waits - bounded - for that number in local memory and copies the slot into a fresh
tensor.  If the wait runs out the kernel records ``BB_STATUS_PEER_TIMEOUT`` and the host
raises ``PeerTimeout``, which the engine maps to its next/previous-stage failure handling.

The host learns the outcome of a receive without synchronising with the stream: a one-thread
kernel behind the receive stores ``(status << 32) | ticket`` into a pinned host word, and the
host polls that word (no driver call on the per-message path).  Like the reference's blocking
``recv``, the engine does not issue work that depends on a message before it has landed.
"""
import ctypes
import json
import time
from datetime import timedelta

import torch

from . import lib as L
from .p2p import ACT, GRAD, PING, PeerTimeout

STATE = 3
_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16, "int64": torch.int64}
_FLAG_BYTES = 8


def _round_up(n, m):
    return (n + m - 1) // m * m


class _InChannel:
    def __init__(self, ptr, flags_bytes, slot_bytes, shape, dtype, nbytes):
        self.ptr, self.flags_bytes, self.slot_bytes = ptr, flags_bytes, slot_bytes
        self.shape, self.dtype, self.nbytes = shape, dtype, nbytes

    def flag(self, i):
        return self.ptr + i * _FLAG_BYTES

    def slot(self, i):
        return self.ptr + self.flags_bytes + i * self.slot_bytes


class _OutChannel(_InChannel):
    counter = None  # 4 bytes of local device memory for the store kernel's last-CTA election


class MailboxTransport:
    name = "mailbox"

    def __init__(self, engine):
        self.rank = engine.global_rank
        self.device = engine.device
        self.store = engine.global_store
        self.slots = engine.micro_batches
        self.timeout_s = engine._config.p2p_timeout_s
        self.blocking = True
        self._in, self._out = {}, {}
        self._lib = L.load()
        # completion record of the latest receive: 8 bytes of pinned host memory the device writes
        host = ctypes.c_void_p()
        L.check(self._lib.bb_pinned_alloc(ctypes.c_longlong(64), ctypes.byref(host)), "bb_pinned_alloc")
        self._done_ptr = host.value
        self._done = ctypes.c_ulonglong.from_address(host.value)
        self._ticket = 0
        # called while the host waits for a message and the stream has drained up to the wait:
        # the engine uses it to issue redundant computation into the otherwise idle GPU
        self.idle_hook = None
        self.measure_idle = False
        self._pre_wait = None
        self.wait_s = 0.0            # host time spent waiting for receives (per-step figure for benchmarks)
        self.idle_s = 0.0            # part of it during which the stream had drained up to the wait

    # ------------------------------------------------------------------ channel set-up
    def _key(self, what, src, dst, kind):
        return f"mbox/{what}/{src}/{dst}/{kind}"

    def _store_get(self, key, peer):
        try:
            self.store.wait([key], timedelta(seconds=self.timeout_s))
            return self.store.get(key)
        except Exception as e:  # store timeout: the peer never reached this channel
            raise PeerTimeout(peer, f"peer rank {peer} did not publish {key}: {str(e)[:120]}")

    def _open_in(self, src, kind, meta):
        """Allocate the local mailbox for (src -> me, kind) and publish its handle."""
        nbytes = _round_up(int(meta["nbytes"]), 16)
        slots = int(meta["slots"])
        flags_bytes = _round_up((slots + 1) * _FLAG_BYTES, 256)
        slot_bytes = _round_up(max(nbytes, 16), 256)
        total = flags_bytes + slots * slot_bytes
        ptr = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        with torch.cuda.device(self.device):
            L.check(self._lib.bb_ipc_alloc(ctypes.c_longlong(total), ctypes.byref(ptr), handle), "bb_ipc_alloc")
        ch = _InChannel(ptr.value, flags_bytes, slot_bytes, tuple(meta["shape"]), _DTYPES[meta["dtype"]], nbytes)
        self._in[(src, kind)] = ch
        self.store.set(self._key("hdl", src, self.rank, kind), bytes(handle))
        return ch

    def _ensure_in(self, src, kind):
        ch = self._in.get((src, kind))
        if ch is None:
            meta = json.loads(self._store_get(self._key("meta", src, self.rank, kind), src).decode())
            ch = self._open_in(src, kind, meta)
        return ch

    def _ensure_out(self, dst, kind, shape, dtype, nbytes, slots):
        ch = self._out.get((dst, kind))
        if ch is not None:
            return ch
        meta = {"shape": list(shape), "dtype": str(dtype).replace("torch.", ""), "nbytes": int(nbytes), "slots": slots}
        self.store.set(self._key("meta", self.rank, dst, kind), json.dumps(meta))
        handle = self._store_get(self._key("hdl", self.rank, dst, kind), dst)
        ptr = ctypes.c_void_p()
        buf = (ctypes.c_ubyte * 64).from_buffer_copy(bytes(handle)[:64])
        with torch.cuda.device(self.device):
            L.check(self._lib.bb_ipc_open(buf, ctypes.byref(ptr)), "bb_ipc_open")
        nb = _round_up(int(nbytes), 16)
        ch = _OutChannel(ptr.value, _round_up((slots + 1) * _FLAG_BYTES, 256), _round_up(max(nb, 16), 256), tuple(shape),
                         dtype, nb)
        ch.counter = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._out[(dst, kind)] = ch
        return ch

    # ------------------------------------------------------------------ data path
    def _stream(self):
        return L._stream()

    def _put(self, ch, slot, src_ptr, nbytes, seq):
        L.LAUNCHES += 1
        L.check(self._lib.bb_p2p_put(ctypes.c_void_p(ch.slot(slot)), ctypes.c_void_p(src_ptr), ctypes.c_longlong(nbytes),
                                     ctypes.c_void_p(ch.flag(slot)), ctypes.c_ulonglong(seq),
                                     ctypes.c_void_p(ch.counter.data_ptr()), self._stream()), "bb_p2p_put")

    def _wait_copy(self, ch, slot, dst_ptr, nbytes, seq):
        L.LAUNCHES += 1
        L.check(self._lib.bb_p2p_wait_copy(ctypes.c_void_p(ch.slot(slot)), ctypes.c_void_p(dst_ptr),
                                           ctypes.c_longlong(nbytes), ctypes.c_void_p(ch.flag(slot)),
                                           ctypes.c_ulonglong(seq), ctypes.c_ulonglong(int(self.timeout_s * 1e9)), None,
                                           self._stream()), "bb_p2p_wait_copy")

    def _finish_recv(self, peer):
        """Wait on the host until the receive kernel retired and turn a recorded timeout into
        an exception (the reference's receives are blocking too).  The wait polls the pinned
        completion word; it gives up a little after the device-side limit."""
        if not self.blocking:
            return
        self._ticket = (self._ticket + 1) & 0xFFFFFFFF or 1
        ticket = self._ticket
        L.LAUNCHES += 1
        L.check(self._lib.bb_p2p_notify(ctypes.c_void_p(self._done_ptr), ctypes.c_uint(ticket), self._stream()),
                "bb_p2p_notify")
        done = self._done
        t0 = time.perf_counter()
        limit = t0 + 2.0 * self.timeout_s + 30.0
        spins = 0
        hook, pre = self.idle_hook, self._pre_wait
        self._pre_wait = None
        drained_at = None
        while True:
            v = done.value
            if (v & 0xFFFFFFFF) == ticket:
                break
            spins += 1
            if pre is not None and (spins & 0x1F) == 0 and (drained_at is not None or pre.query()):
                # everything queued before the wait has run: the stream now sits in the wait kernel
                if drained_at is None:
                    drained_at = time.perf_counter()
                if hook is not None and not hook(idle_for_s=time.perf_counter() - drained_at):
                    hook = None
            if (spins & 0xFFF) == 0 and time.perf_counter() > limit:
                raise L.BambooNativeError(f"no completion record for a receive from rank {peer} "
                                          f"after {2.0 * self.timeout_s + 30.0:.0f} s")
        now = time.perf_counter()
        self.wait_s += now - t0
        if drained_at is not None:
            self.idle_s += now - drained_at      # the GPU's own-stage stream had nothing but the wait
        status = v >> 32
        if status == 0:
            return
        torch.cuda.current_stream(self.device).synchronize()
        L.read_status()                      # clears the device word
        if status == L.STATUS_PEER_TIMEOUT:
            raise PeerTimeout(peer)
        raise L.BambooNativeError(f"device status {status} after a receive from rank {peer}")

    def send(self, tensor, dst, kind, slot, seq):
        t = tensor.detach()
        if not t.is_contiguous():
            t = t.contiguous()
        nbytes = t.numel() * t.element_size()
        ch = self._ensure_out(dst, kind, t.shape, t.dtype, nbytes, self.slots)
        if tuple(t.shape) != ch.shape or t.dtype != ch.dtype:
            raise L.BambooNativeError(f"message geometry changed on channel to rank {dst}: {tuple(t.shape)} vs {ch.shape}")
        if nbytes % 16:
            pad = torch.zeros(ch.nbytes, dtype=torch.uint8, device=t.device)
            pad[:nbytes].copy_(t.view(torch.uint8).reshape(-1))
            t = pad
        self._put(ch, slot, t.data_ptr(), ch.nbytes, seq)
        self._keep = t  # the store kernel reads it asynchronously; stream order frees it safely

    def recv(self, src, kind, slot, seq):
        ch = self._ensure_in(src, kind)
        numel = 1
        for d in ch.shape:
            numel *= d
        raw = torch.empty(ch.nbytes, dtype=torch.uint8, device=self.device)
        if self.idle_hook is not None or self.measure_idle:
            self._pre_wait = torch.cuda.Event()
            self._pre_wait.record()
        self._wait_copy(ch, slot, raw.data_ptr(), ch.nbytes, seq)
        self._finish_recv(src)
        esz = torch.empty(0, dtype=ch.dtype).element_size()
        return raw[: numel * esz].view(ch.dtype).view(ch.shape)

    def send_ping(self, dst, seq):
        ch = self._ensure_out(dst, PING, (0,), torch.float32, 0, 1)
        L.LAUNCHES += 1
        L.check(self._lib.bb_p2p_signal(ctypes.c_void_p(ch.flag(0)), ctypes.c_ulonglong(seq), self._stream()),
                "bb_p2p_signal")

    def recv_ping(self, src, seq):
        ch = self._ensure_in(src, PING)
        self._wait_copy(ch, 0, 0, 0, seq)
        self._finish_recv(src)

    def exchange_state(self, send_to, tensors_out, recv_from, tensors_in, seq):
        """End-of-step shadow refresh: every piece travels through a staging mailbox on the
        receiver and is then copied into its shadow arena."""
        seq = int(seq)
        if recv_from is not None and (recv_from, STATE) not in self._in:
            # the receiver knows the size (its shadow arena), so it can publish first and
            # nobody waits in a cycle around the stage ring
            sizes = [t.numel() * t.element_size() for t in tensors_in]
            self._open_in(recv_from, STATE, {"shape": [0], "dtype": "float32", "nbytes": max(sizes), "slots": len(sizes)})
        if send_to is not None:
            sizes = [t.numel() * t.element_size() for t in tensors_out]
            ch = self._ensure_out(send_to, STATE, (0,), torch.float32, max(sizes), len(sizes))
            for i, t in enumerate(tensors_out):
                self._put(ch, i, t.data_ptr(), _round_up(t.numel() * t.element_size(), 16), seq)
        if recv_from is not None:
            # all pieces or none: the kernel copies only after every piece's flag has arrived
            ch = self._in[(recv_from, STATE)]
            n = len(tensors_in)
            slots = (ctypes.c_void_p * n)(*[ch.slot(i) for i in range(n)])
            dsts = (ctypes.c_void_p * n)(*[t.data_ptr() for t in tensors_in])
            sizes = (ctypes.c_longlong * n)(*[_round_up(t.numel() * t.element_size(), 16) for t in tensors_in])
            L.LAUNCHES += 1
            L.check(self._lib.bb_p2p_wait_copy_multi(slots, dsts, sizes, ctypes.c_int(n), ctypes.c_void_p(ch.flag(0)),
                                                     ctypes.c_ulonglong(seq), ctypes.c_ulonglong(int(self.timeout_s * 1e9)),
                                                     None, self._stream()), "bb_p2p_wait_copy_multi")
            self._finish_recv(recv_from)

    def forget_peer(self, peer):
        for table in (self._in, self._out):
            for key in [k for k in table if k[0] == peer]:
                table.pop(key)  # mappings of a dead peer are left to process teardown

    def end_step(self):
        return

    def close(self):
        torch.cuda.synchronize(self.device)
        if self._done_ptr:
            self._done = None
            self._lib.bb_pinned_free(ctypes.c_void_p(self._done_ptr))
            self._done_ptr = 0
