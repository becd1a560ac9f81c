"""N-column sharding of the fused LM head over the GPUs of one node.

Every rank holds its own re-packed NVFP4 shard `[K, 9 * N_r / 16]` (a column shard is not a
contiguous slice of the packed tensor, see packing.nvfp4_column_slice) and the replicated
activations.  One step is: the fused SkinnyGemm + ArgmaxRows kernel over the local columns,
which emits per row a 64-bit key ordering (value, global index) pairs exactly like ArgmaxRows;
the exchange of those keys (8 bytes per row per rank) - on GPUs inside the fused kernel, whose last
CTA stores them into every rank's peer-mapped buffer and folds what arrives, else one all-gather
followed by a fold kernel.  Larger key = better pair: larger value, then lower index; NaN above all.

The reference has no distributed code; the vocabulary projection is the one op of the path whose
columns can be split over the GPUs of a node with a single small exchange.
"""
from __future__ import annotations

import numpy as np

from . import packing


def pack_key(val: np.ndarray, idx: np.ndarray) -> np.ndarray:
    """Host restatement of the key the kernel emits, for checking gathered payloads."""
    v = np.asarray(val, dtype=np.float32).copy()
    v[v == 0] = 0.0  # -0 and +0 compare equal
    b = v.view(np.uint32).astype(np.uint64)
    ord_ = np.where(b & 0x80000000, (~b) & 0xFFFFFFFF, b | 0x80000000)
    ord_ = np.where(np.isnan(v), np.uint64(0xFFFFFFFF), ord_)
    return (ord_.astype(np.uint64) << np.uint64(32)) | (np.uint64(0xFFFFFFFF) - np.asarray(idx, dtype=np.uint64))


def unpack_key(key: np.ndarray):
    key = np.asarray(key).view(np.uint64) if np.asarray(key).dtype != np.uint64 else np.asarray(key)
    ord_ = (key >> np.uint64(32)).astype(np.uint32)
    bits = np.where(ord_ & 0x80000000, ord_ & 0x7FFFFFFF, ~ord_).astype(np.uint32)
    bits = np.where(ord_ == 0xFFFFFFFF, np.uint32(0x7FC00000), bits)
    idx = (np.uint64(0xFFFFFFFF) - (key & np.uint64(0xFFFFFFFF))).astype(np.int64)
    return bits.view(np.float32), idx


def fold_keys_host(keys: np.ndarray):
    """[ranks, m] gathered keys -> (idx, val); the host mirror of the device fold."""
    best = np.asarray(keys).view(np.uint64).reshape(keys.shape).max(axis=0)
    val, idx = unpack_key(best)
    return idx, val


class PeerExchange:
    """This rank's exchange buffer and its mappings of the other ranks' buffers (CUDA IPC handles passed
    around with torch.distributed).  Set-up allocates and synchronises; steps do neither."""

    def __init__(self, group=None):
        import ctypes

        import torch.distributed as dist

        from . import _lib

        lib = _lib.load()
        self._lib = lib
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.own = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        _lib.check(lib.qfg_peer_alloc(lib.qfg_lmhead_exchange_bytes(), ctypes.byref(self.own), handle))
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self.struct = _lib.LmExchange()
        self.struct.world, self.struct.rank = self.world, self.rank
        self._opened = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.struct.peers[r] = self.own.value
            else:
                ptr = ctypes.c_void_p()
                _lib.check(lib.qfg_peer_open(ctypes.create_string_buffer(h, 64), ctypes.byref(ptr)))
                self._opened.append(ptr)
                self.struct.peers[r] = ptr.value
        dist.barrier(group=group)  # nobody steps before every mapping exists

    def status(self) -> int:
        import ctypes

        from . import _lib

        s = ctypes.c_int(0)
        _lib.check(self._lib.qfg_lmhead_exchange_status(self.own, ctypes.byref(s)))
        return s.value

    def times(self):
        """Device timer (ns) of this rank's last sharded call: (keys ready, stores to the peers issued, all
        ranks' words seen).  Synchronises the device."""
        import ctypes

        from . import _lib

        t = (ctypes.c_uint64 * 3)()
        _lib.check(self._lib.qfg_lmhead_exchange_times(self.own, t))
        return int(t[0]), int(t[1]), int(t[2])

    def close(self):
        for ptr in self._opened:
            self._lib.qfg_peer_close(ptr)
        self._opened = []
        if self.own:
            self._lib.qfg_peer_free(self.own)
            self.own = None


class ShardedLmHead:
    """One rank of the N-sharded LM head.

    `shard` is this rank's packed weight (CUDA uint8 tensor [K, 9 * n_local / 16]) covering global
    columns [col_begin, col_begin + n_local).  `group` is a torch.distributed process group (NCCL
    for CUDA tensors); with world size 1 no collective is issued.
    """

    def __init__(self, shard, n_local: int, col_begin: int, group=None, w_scale=None, exchange: str = "auto"):
        import torch
        import torch.distributed as dist

        from .ops import LmHeadArgmax

        self.shard = shard
        self.n_local = int(n_local)
        self.col_begin = int(col_begin)
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.head = LmHeadArgmax(w_scale=w_scale, device=shard.device)
        self._torch = torch
        self._dist = dist
        self._gathered = None
        # "peer": keys exchanged inside the fused kernel through peer memory; "nccl": all-gather + fold kernel;
        # "auto": peer memory on CUDA when the mappings can be set up, else NCCL
        self.peer = None
        if self.world > 1 and exchange in ("auto", "peer") and shard.is_cuda:
            try:
                self.peer = PeerExchange(group)
            except Exception:
                if exchange == "peer":
                    raise
                self.peer = None
            # every rank must take the same path
            ok = torch.tensor([1 if self.peer is not None else 0], device=shard.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if int(ok.item()) == 0:
                if self.peer is not None:
                    self.peer.close()
                self.peer = None

    @staticmethod
    def column_range(n_total: int, rank: int, world: int, granule: int = 128):
        return packing.shard_columns(n_total, world, granule)[rank]

    def step(self, x, checked: bool = False):
        """x: BF16 [m, K] on this rank's GPU (replicated).  Returns (idx int64 [m], val float32 [m]),
        identical on every rank.  `checked` (peer-memory exchange only): synchronise and raise if a wait for a
        peer's keys ran out, in which case the ranks may hold different winners."""
        from .ops import lmhead_combine

        torch = self._torch
        if self.peer is not None:
            out = self.head.call_sharded(x, self.shard, self.n_local, self.col_begin, self.peer.struct)
            if checked and self.peer.status() != 0:
                from ._lib import QFG_FAIL, QfgError

                raise QfgError(QFG_FAIL, "LmHead: the wait for a peer's keys ran out; the result lacks that peer")
            return out
        idx, val, key = self.head(x, self.shard, self.n_local, col_offset=self.col_begin)
        if self.world == 1:
            return idx, val
        m = key.numel()
        if self._gathered is None or self._gathered.numel() != self.world * m:
            self._gathered = torch.empty(self.world * m, dtype=torch.int64, device=key.device)
        self._dist.all_gather_into_tensor(self._gathered, key, group=self.group)
        return lmhead_combine(self._gathered, self.world, m)


class HostLmHead:
    """The LM head for a caller whose activations and results live in host memory.

    One call copies `x` (pinned host, BF16 [m, K]) to the device, runs the sharded step and leaves the
    winning index and value in pinned host buffers.  Whenever the step is a single kernel (one GPU, or
    several ranks exchanging their keys through peer memory inside the kernel) the call is
    qfg_lmhead_host_run: a CUDA graph, recorded once by the library, of the input copy and the fused
    kernel, which stores its results straight into the pinned host buffers; a call then costs one
    graph launch and one stream synchronisation.  With the NCCL exchange the stages are issued eagerly
    around the all-gather.  Every rank must construct the object and make its calls in step with the
    others.
    """

    def __init__(self, head: ShardedLmHead, m: int, k: int):
        import ctypes

        from . import _lib
        from .ops import _tensor2d

        torch = head._torch
        dev = head.shard.device
        self.head = head
        self.x_host = torch.empty((m, k), dtype=torch.bfloat16).pin_memory()
        self.x_dev = torch.empty((m, k), dtype=torch.bfloat16, device=dev)
        self.idx_host = torch.empty(m, dtype=torch.int64).pin_memory()
        self.val_host = torch.empty(m, dtype=torch.float32).pin_memory()
        self._lib = _lib.load()
        self._h = None
        self.stream = None
        if head.world == 1 or head.peer is not None:
            t = _tensor2d(head.shard)
            exchange = ctypes.byref(head.peer.struct) if head.peer is not None else None
            h = ctypes.c_void_p()
            with torch.cuda.device(dev):
                torch.cuda.synchronize()  # the workspace clear and anything else queued by torch precedes the first step
                _lib.check(self._lib.qfg_lmhead_host_create(
                    head.head._h, m, k, ctypes.byref(t), head.n_local, head.col_begin, head.head.workspace.data_ptr(),
                    exchange, self.x_host.data_ptr(), self.x_dev.data_ptr(), self.idx_host.data_ptr(),
                    self.val_host.data_ptr(), ctypes.byref(h)))
            self._h = h
        else:
            self.stream = torch.cuda.Stream(device=dev)

    def __call__(self, x_host=None):
        """x_host: optional BF16 [m, K] host tensor to stage first (omit when the caller wrote
        `self.x_host` in place).  Returns (idx_host, val_host), valid until the next call."""
        if x_host is not None:
            self.x_host.copy_(x_host)
        if self._h is not None:
            rc = self._lib.qfg_lmhead_host_run(self._h)
            if rc != 0:
                from . import _lib

                _lib.check(rc)
            return self.idx_host, self.val_host
        torch = self.head._torch
        with torch.cuda.stream(self.stream):
            self.x_dev.copy_(self.x_host, non_blocking=True)
            idx, val = self.head.step(self.x_dev)
            self.idx_host.copy_(idx, non_blocking=True)
            self.val_host.copy_(val, non_blocking=True)
        self.stream.synchronize()
        return self.idx_host, self.val_host

    def __del__(self):
        h = getattr(self, "_h", None)
        if h is not None:
            self._lib.qfg_lmhead_host_destroy(h)
            self._h = None
