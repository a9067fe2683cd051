"""Expert-parallel row exchange with peer stores over NVLink.

`PeerExchange` owns one symmetric allocation per process group (torch.distributed._symmetric_memory: the same
buffer mapped on every GPU of the group), split into a flag array and a few receive regions. An exchange is two
kernels of libffmoe on the current stream: `ffm_p2p_push` stores this rank's row segments straight into the peers'
receive regions, `ffm_p2p_signal_wait` publishes an epoch flag to every peer and waits (bounded) for theirs. All
offsets come from the [ep, ep] matrix of row counts every rank already knows, so nothing but rows and flags crosses
NVLink. No multicast object is bound (TORCH_SYMM_MEM_DISABLE_MULTICAST=1) and no multimem instruction is used.

Region reuse needs no extra barrier as long as a rank has consumed (or copied) a region, in stream order, before it
signals the exchange after which a peer may push into that region again. The forward pass alternates regions 0 and
1, so this holds by construction; rows of a backward exchange are read in place after its barrier, so consecutive
backward exchanges alternate between regions 2 and 3 (fused_moe._backward_region).
"""

import ctypes
import os

import numpy as np
import torch

from . import _lib, ops

# Head of the symmetric buffer: [0, 2048) flags of the host-epoch barrier, [2048, 3072) flags of the device-epoch
# barrier, [3072, 3076) its epoch counter, [4096, 4096 + 16 KiB) the [ep, E] int32 count matrix of the host-sync-free
# forward (every rank writes its row into every rank's copy).
FLAG_BYTES = 65536
DEV_FLAGS_OFFSET = 2048
DEV_COUNTER_OFFSET = 3072
COUNTS_OFFSET = 4096
COUNTS_BYTES = 16 * 256 * 4
# dispatch, combine (also the reverse-dispatch of the full input gradient), and two backward regions used in turn
NUM_REGIONS = 4

_exchanges = {}


class SegmentPlan:
    """Row runs of one expert-parallel call between every sender's expert-sorted order and every receiver's grouped
    layout, from the [ep, E] matrix C[s][e] = rows rank s routes to expert e (host integers, same on every rank).

    Sender order (rank s): its routed rows sorted by expert, no padding; expert e starts at row send0[s][e].
    Receiver layout (rank d, experts d*El .. (d+1)*El-1): expert segments aligned to 256 rows (tile_start in 128-row
    tiles, as the grouped GEMM expects); inside a segment the rows of source rank 0 come first, then rank 1, ...;
    the run of (source s, expert e) starts at row recv0[s][e] of rank (e // El).
    Tables (int64 [n, 4] = {first source row, first destination row, rows, destination rank}, plus running ends):
      dispatch  this rank's runs, sender order -> receivers' grouped layouts
      combine   the runs this rank holds as expert owner, grouped layout -> the origins' sender order
      padding   the rows between a segment's last row and the next segment of this rank's own layout (to be zeroed)
    """

    def __init__(self, C, e_local, rank):
        C = np.asarray(C, dtype=np.int64)
        ep, E = C.shape
        assert E == ep * e_local
        self.ep, self.e_local, self.rank = ep, e_local, rank
        self.send0 = np.cumsum(C, axis=1) - C                       # [ep, E]
        self.send_rows = C.sum(axis=1)                              # rows every rank sends (= its T)
        R = C.sum(axis=0)                                           # rows per expert over all sources
        tiles = 2 * ((R + 255) // 256)                              # 128-row tiles per expert segment, even
        tiles_l = tiles.reshape(ep, e_local)
        ts = np.zeros((ep, e_local + 1), dtype=np.int64)
        ts[:, 1:] = np.cumsum(tiles_l, axis=1)
        self.tile_start = ts                                        # [ep, El + 1] per destination rank
        self.rows_grouped = ts[:, -1] * 128                         # grouped rows (with padding) per rank
        self.recv_rows = R.reshape(ep, e_local).sum(axis=1)         # valid rows per rank (M)
        seg0 = (ts[:, :-1] * 128).reshape(E)                        # first row of expert e's segment at its owner
        self.recv0 = seg0[None, :] + (np.cumsum(C, axis=0) - C)     # [ep, E]
        owner = np.arange(E) // e_local
        r = rank
        mine = np.nonzero(C[r] > 0)[0]
        self.dispatch = self._table(self.send0[r, mine], self.recv0[r, mine], C[r, mine], owner[mine])
        lo, hi = r * e_local, (r + 1) * e_local
        sub = C[:, lo:hi]                                           # [ep, El] rows this rank receives
        e_idx, s_idx = np.nonzero(sub.T > 0)                        # expert-major, source within expert
        self.combine = self._table(self.recv0[s_idx, lo + e_idx], self.send0[s_idx, lo + e_idx], sub[s_idx, e_idx], s_idx)
        end_valid = seg0[lo:hi] + R[lo:hi]
        end_seg = ts[r, 1:] * 128
        pad = end_seg - end_valid
        has = np.nonzero(pad > 0)[0]
        self.padding = self._table(np.zeros(len(has), dtype=np.int64), end_valid[has], pad[has],
                                   np.full(len(has), r, dtype=np.int64))

    @staticmethod
    def _table(src0, dst0, rows, dst_rank):
        seg = np.stack([src0, dst0, rows, dst_rank], axis=1).astype(np.int64).reshape(-1, 4)
        return seg, np.cumsum(seg[:, 2]).astype(np.int64)


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
        self._dev_flag_ptrs = (ctypes.c_void_p * self.world)(*[p + DEV_FLAGS_OFFSET for p in self.ptrs])

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

    def upload(self, *arrays):
        """One host -> device copy for several int64 tables; returns device views in the same order."""
        flat = np.concatenate([np.ascontiguousarray(a, dtype=np.int64).reshape(-1) for a in arrays])
        if flat.size == 0:
            flat = np.zeros(1, dtype=np.int64)
        dev = torch.from_numpy(flat).pin_memory().to(self.buf.device, non_blocking=True)
        out, o = [], 0
        for a in arrays:
            n = int(np.asarray(a).size)
            out.append(dev[o:o + n])
            o += n
        return out


    def push_rows(self, src, src_index, index_div, row_bytes, seg_dev, end_dev, n_segments, total_rows, region,
                          remote_rows=0, dry=False, name="all_to_all"):
        """Row runs listed in a device table (ffm_p2p_push_rows) into region `region` of the ranks named by the table.
        src None zeroes the rows. remote_rows only feeds the byte counter."""
        if n_segments == 0 or total_rows == 0 or dry:
            return
        lib = _lib.load()
        n = self.world
        bases = (ctypes.c_void_p * n)(*[self.region_ptr(d, region) for d in range(n)])
        ops.a2a_bytes_sent += remote_rows * row_bytes
        with ops._Launch(name, 1, also="exchange_rows" if name == "all_to_all" else None):
            _lib.check(lib.ffm_p2p_push_rows(0 if src is None else src.data_ptr(),
                                             0 if src_index is None else src_index.data_ptr(), int(index_div),
                                             int(row_bytes), seg_dev.data_ptr(), end_dev.data_ptr(), int(n_segments),
                                             int(total_rows), bases, n, ops._stream()), "ffm_p2p_push_rows")


    def barrier(self, dry=False):
        """Flag barrier of the group on the current stream: what the peers pushed before it is readable after it."""
        if dry:
            return
        lib = _lib.load()
        self.epoch += 1
        with ops._Launch("all_to_all", 1):
            _lib.check(lib.ffm_p2p_signal_wait(self._flag_ptrs, self.rank, self.world, self.epoch,
                                               ops.status_tensor(self.buf.device).data_ptr(), 0, ops._stream()),
                       "ffm_p2p_signal_wait")


    def barrier_dev(self):
        """Flag barrier whose epoch lives in device memory (replayable inside a CUDA graph)."""
        lib = _lib.load()
        with ops._Launch("all_to_all", 1):
            _lib.check(lib.ffm_p2p_signal_wait_dev(self._dev_flag_ptrs, self.rank, self.world,
                                                   self.ptrs[self.rank] + DEV_COUNTER_OFFSET,
                                                   ops.status_tensor(self.buf.device).data_ptr(), 0, ops._stream()),
                       "ffm_p2p_signal_wait_dev")

    def share_counts(self, counts):
        """counts int32 [E] of this rank -> row `rank` of every rank's [ep, E] count matrix; returns this rank's copy
        (valid after the barrier this call ends with; no host involvement)."""
        lib = _lib.load()
        E = counts.numel()
        n = self.world
        if E * 4 % 16 != 0 or n * E * 4 > COUNTS_BYTES:
            raise RuntimeError("share_counts needs E % 4 == 0 and ep * E <= 4096")
        src = (ctypes.c_void_p * n)(*[counts.data_ptr()] * n)
        dst = (ctypes.c_void_p * n)(*[p + COUNTS_OFFSET + self.rank * E * 4 for p in self.ptrs])
        nbytes = (ctypes.c_int64 * n)(*[E * 4] * n)
        with ops._Launch("all_to_all", 1):
            _lib.check(lib.ffm_p2p_push(n, src, dst, nbytes, ops._stream()), "ffm_p2p_push")
        self.barrier_dev()
        return self.buf[COUNTS_OFFSET:COUNTS_OFFSET + n * E * 4].view(torch.int32).view(n, E)

    def plan_dev(self, count_matrix, e_local, max_grouped_rows=0):
        """Device-built tables of one call (ffm_p2p_plan) from the shared count matrix. max_grouped_rows > 0: the
        rows every rank's receive buffer holds; if any rank's grouped layout would exceed it the tables move nothing
        and the status word gets FFM_STATUS_EP_OVERFLOW."""
        lib = _lib.load()
        ep = self.world
        E = ep * e_local
        dev = self.buf.device
        i64 = dict(dtype=torch.int64, device=dev)
        t = dict(dispatch=torch.empty(E, 4, **i64), dispatch_end=torch.empty(E, **i64),
                 combine=torch.empty(e_local * ep, 4, **i64), combine_end=torch.empty(e_local * ep, **i64),
                 padding=torch.empty(e_local, 4, **i64), padding_end=torch.empty(e_local, **i64),
                 tile_start=torch.empty(e_local + 1, dtype=torch.int32, device=dev), totals=torch.empty(4, **i64))
        with ops._Launch("ep_plan", 1):
            _lib.check(lib.ffm_p2p_plan(count_matrix.data_ptr(), ep, e_local, self.rank, t["dispatch"].data_ptr(),
                                        t["dispatch_end"].data_ptr(), t["combine"].data_ptr(),
                                        t["combine_end"].data_ptr(), t["padding"].data_ptr(),
                                        t["padding_end"].data_ptr(), t["tile_start"].data_ptr(),
                                        t["totals"].data_ptr(), int(max_grouped_rows),
                                        ops.status_tensor(dev).data_ptr(), ops._stream()), "ffm_p2p_plan")
        return t

    def push_rows_dev(self, src, src_index, index_div, row_bytes, seg, seg_end, total_dev, max_rows, region,
                      name="all_to_all"):
        """push_rows with the row total read on the device (tables from plan_dev)."""
        lib = _lib.load()
        n = self.world
        bases = (ctypes.c_void_p * n)(*[self.region_ptr(d, region) for d in range(n)])
        with ops._Launch(name, 1, also="exchange_rows" if name == "all_to_all" else None):
            _lib.check(lib.ffm_p2p_push_rows_dev(0 if src is None else src.data_ptr(),
                                                 0 if src_index is None else src_index.data_ptr(), int(index_div),
                                                 int(row_bytes), seg.data_ptr(), seg_end.data_ptr(), int(seg.shape[0]),
                                                 total_dev.data_ptr(), int(max_rows), bases, n, ops._stream()),
                       "ffm_p2p_push_rows_dev")

    def keep_rows_dev(self, src, rows_dev, max_rows):
        """A copy of the first *rows_dev rows of `src` ([max_rows, W]; the count is an int64 [1] device tensor) in a
        new tensor of the same shape; the rows beyond the count stay uninitialised. Costs what the rows in use cost,
        whatever the worst-case size of the buffer."""
        lib = _lib.load()
        dst = torch.empty_like(src)
        if not hasattr(self, "_self_copy_head"):
            self._self_copy_head = torch.zeros(2, dtype=torch.int64, device=self.buf.device)
            self._self_copy_rank = torch.full((1,), self.rank, dtype=torch.int64, device=self.buf.device)
        rows_dev = rows_dev.reshape(1)
        seg = torch.cat([self._self_copy_head, rows_dev, self._self_copy_rank])   # {src row 0, dst row 0, rows, self}
        n = self.world
        bases = (ctypes.c_void_p * n)(*[dst.data_ptr()] * n)
        with ops._Launch("keep_rows", 1):
            _lib.check(lib.ffm_p2p_push_rows_dev(src.data_ptr(), 0, 1, int(src.shape[1] * src.element_size()),
                                                 seg.data_ptr(), rows_dev.data_ptr(), 1, rows_dev.data_ptr(),
                                                 int(max_rows), bases, n, ops._stream()), "ffm_p2p_push_rows_dev")
        return dst

    def region_view(self, region, rows, width, dtype):
        lo = FLAG_BYTES + region * self.region_bytes
        nbytes = rows * width * torch.empty(0, dtype=dtype).element_size()
        return self.buf[lo:lo + nbytes].view(dtype).view(rows, width)



def get_exchange(group, device, region_bytes):
    """One PeerExchange per (group, device), grown (collectively) when a larger region is asked for."""
    key = (id(group), torch.device(device).index)
    px = _exchanges.get(key)
    if px is None or px.region_bytes < region_bytes:
        old = px
        px = PeerExchange(group, device, region_bytes)   # (its constructor ends with a group barrier)
        _exchanges[key] = px
        if old is not None:
            # Let go of the smaller buffer: every rank has left its last exchange on it (it took part in the new
            # buffer's rendezvous and barrier after it), and tensors that still view it keep its storage alive.
            old.buf = old.hdl = None
            old.ptrs = []
    return px
