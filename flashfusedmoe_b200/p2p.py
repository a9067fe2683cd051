"""Expert-parallel row exchange with peer stores over NVLink.

`PeerExchange` owns one symmetric allocation per process group (torch.distributed._symmetric_memory: the same
buffer mapped on every GPU of the group), split into a flag array and a few receive regions. An exchange is two
kernels of libffmoe on the current stream: `ffm_p2p_push` stores this rank's row segments straight into the peers'
receive regions, `ffm_p2p_signal_wait` publishes an epoch flag to every peer and waits (bounded) for theirs. All
offsets come from the [ep, ep] matrix of row counts every rank already knows, so nothing but rows and flags crosses
NVLink. No multicast object is bound (TORCH_SYMM_MEM_DISABLE_MULTICAST=1) and no multimem instruction is used.

Region reuse is safe without extra barriers because every exchange is a full barrier of the group and the layer
consumes (or copies) a region before it takes part in the exchange that could overwrite it.
"""

import ctypes
import os

import torch

from . import _lib, ops

FLAG_BYTES = 4096
NUM_REGIONS = 3  # dispatch, combine (also the reverse-dispatch of the full input gradient), backward

_exchanges = {}


def available():
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
        return True
    except Exception:
        return False


class PeerExchange:
    def __init__(self, group, device, region_bytes):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > 16:
            raise RuntimeError("PeerExchange supports at most 16 ranks (FFM_P2P_MAX_PEERS)")
        self.region_bytes = (int(region_bytes) + 255) // 256 * 256
        total = FLAG_BYTES + NUM_REGIONS * self.region_bytes
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.buf[:FLAG_BYTES].zero_()
        self.hdl = symm_mem.rendezvous(self.buf, group)
        self.ptrs = [int(p) for p in self.hdl.buffer_ptrs]
        torch.cuda.synchronize(device)
        dist.barrier(group)  # every rank's flags are zero before anyone signals
        self.epoch = 0
        self._flag_ptrs = (ctypes.c_void_p * self.world)(*self.ptrs)

    def region_ptr(self, rank, region):
        return self.ptrs[rank] + FLAG_BYTES + region * self.region_bytes

    def fits(self, max_rows, row_bytes):
        return max_rows * row_bytes <= self.region_bytes

    def exchange(self, rows, counts, region, dry=False):
        """rows [sum_d counts[rank][d], W] ordered by destination; counts[s][d] = rows rank s sends to rank d
        (host lists, identical on every rank). Returns a [M, W] view of this rank's receive region, valid until the
        next exchange that uses the same region. dry=True (measurement aid) launches nothing and returns the view."""
        lib = _lib.load()
        W = rows.shape[1]
        row_bytes = W * rows.element_size()
        r, n = self.rank, self.world
        if dry:
            M = sum(counts[s][r] for s in range(n))
            lo = FLAG_BYTES + region * self.region_bytes
            return self.buf[lo:lo + M * row_bytes].view(rows.dtype).view(M, W)
        src = (ctypes.c_void_p * n)()
        dst = (ctypes.c_void_p * n)()
        nbytes = (ctypes.c_int64 * n)()
        send_off = 0
        base = rows.data_ptr()
        for d in range(n):
            cnt = counts[r][d]
            recv_off = sum(counts[s][d] for s in range(r))
            src[d] = base + send_off * row_bytes
            dst[d] = self.region_ptr(d, region) + recv_off * row_bytes
            nbytes[d] = cnt * row_bytes
            send_off += cnt
        ops.a2a_bytes_sent += (send_off - counts[r][r]) * row_bytes
        M = sum(counts[s][r] for s in range(n))
        stream = ops._stream()
        with ops._Launch("all_to_all", 2):
            if send_off > 0:
                _lib.check(lib.ffm_p2p_push(n, src, dst, nbytes, stream), "ffm_p2p_push")
            self.epoch += 1
            _lib.check(lib.ffm_p2p_signal_wait(self._flag_ptrs, r, n, self.epoch,
                                               ops.status_tensor(rows.device).data_ptr(), 0, stream),
                       "ffm_p2p_signal_wait")
        lo = FLAG_BYTES + region * self.region_bytes
        return self.buf[lo:lo + M * row_bytes].view(rows.dtype).view(M, W)


def get_exchange(group, device, region_bytes):
    """One PeerExchange per (group, device), grown (collectively) when a larger region is asked for."""
    key = (id(group), torch.device(device).index)
    px = _exchanges.get(key)
    if px is None or px.region_bytes < region_bytes:
        px = PeerExchange(group, device, region_bytes)
        _exchanges[key] = px
    return px
