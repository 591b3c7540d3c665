"""Multi-GPU partitioning of the fused embedding-bag forward (one process per GPU, torch.distributed).

The reference has no multi-GPU data path (it uses several GPUs only as independent tuning workers,
RecFlex/tuning/measure.py:27,68); both modes here are new:

* replicated tables, batch split: every rank holds all tables and pools its own share of the samples
  with the plain `FeatEmbed`; nothing is exchanged.  Nothing to add beyond `FeatEmbed`.
* table-wise sharding (`plan_shards` + `ShardedFeatEmbed`): whole tables are assigned to ranks by a
  size/traffic-balanced planner; each rank pools ITS features for the WHOLE batch, the pooled rows are
  exchanged with one all-to-all per batch chunk over NCCL (NVLink/NVSwitch), and a placement kernel puts
  every feature's columns at its canonical position, so that rank r ends with `[B / world, sum(dim)]` for
  its share of the samples, identical to what the unsharded module computes for those samples.

Three exchanges are implemented.  `exchange="peer"` is the fused one: the outputs of all ranks live in buffers
every rank has mapped (CUDA IPC over NVLink), and the fused kernel stores each pooled row straight into the
destination rank's final matrix at the feature's canonical columns, so the transfer overlaps the pooling tile by
tile and no send buffer, all-to-all or placement pass exists; a one-element all-reduce on the same stream tells
every rank that all kernels are done.  It hides the transfer completely at 2 and 4 GPUs.  `exchange="copy"` is for
8 GPUs, where 7/8 of every pooled row leaves the GPU and plain stores of 64 to 512 bytes use NVLink less well than
the copy engines do: the kernel pools into a local send buffer in ONE launch whose tile order walks the batch piece
by piece, and a copy stream ships every finished piece as one 2-D copy per destination (rows of sum(local dims)
elements) while the next piece is pooled (`eb_forward_exchange`).  Its result has the columns grouped by owner rank
(`column_of[f]` says where feature f starts); `columns="blocks"` returns one `[B / world, sum(dims of rank s)]`
tensor per owner rank instead (every copy is then one contiguous run on both sides), and `columns="canonical"` adds a
placement pass that restores feature order.  `exchange="push"` is the copy exchange with the pieces shipped by a small kernel (warps storing 512-byte runs to
the peers) instead of the copy engines.  `exchange="nccl"` is the library baseline: pool into a send buffer, `all_to_all_single`, placement kernel.

With `exchange="nccl"`, batch chunks pipeline the exchange behind the pooling: chunk k's all-to-all runs on a side stream
while chunk k + 1 is pooled.  With C chunks, sample b of the batch belongs to chunk `b // (B / C)` and,
inside the chunk, to rank `(b % (B / C)) // (B / (C * world))`; a rank's output rows are its samples in
batch order.  With the other two exchanges rank r ends with samples `[r, r + 1) * B / world`.

Outputs of the peer and copy exchanges are views of buffers the module owns (two, used in turn): a result is
valid until the call after the next one, and no longer after `close()` or a change of batch size.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import _lib


# ---------------------------------------------------------------------------
# planner
# ---------------------------------------------------------------------------
def plan_shards(table_bytes: Sequence[int], traffic: Sequence[float], world: int,
                capacity_bytes: Optional[int] = None, exchange: Optional[Sequence[float]] = None) -> List[int]:
    """Owner rank of every table.

    Longest-processing-time greedy on `traffic` (expected gathered bytes per batch: nnz_f * row_bytes_f)
    under a per-rank capacity on `table_bytes`, then pairwise moves/swaps while they lower the maximum
    per-rank traffic.  Raises if the tables do not fit.

    `exchange` (optional: bytes of pooled output each table's owner sends per batch, batch * dim_f * 4 * (world - 1) /
    world) adds a second load to balance.  One-hot features produce twice as many output bytes as they gather from
    an fp16 table, so ranks with equal gather traffic can differ by 15 % and more in what they push through NVLink,
    and at 8 GPUs the exchange, not the pooling, bounds the step.  With it the planner minimises the larger of the
    two per-rank loads, each measured against its own mean.
    """
    F = len(table_bytes)
    if len(traffic) != F or world < 1:
        raise ValueError("table_bytes and traffic must have one entry per table, world >= 1")
    cap = capacity_bytes if capacity_bytes is not None else float("inf")
    if any(b > cap for b in table_bytes):
        raise ValueError("a single table exceeds the per-rank capacity")
    if exchange is not None:
        if len(exchange) != F:
            raise ValueError("exchange must have one entry per table")
        return _plan_two_loads(table_bytes, traffic, exchange, world, cap)
    owner = [-1] * F
    load = [0.0] * world
    used = [0] * world
    # heaviest traffic first; among equals the bigger table first (harder to place)
    for f in sorted(range(F), key=lambda i: (-traffic[i], -table_bytes[i])):
        ranks = [r for r in range(world) if used[r] + table_bytes[f] <= cap]
        if not ranks:
            # make room: capacity-aware fallback = rank with the most free bytes must fit it
            raise ValueError("tables do not fit the per-rank capacity with this greedy order; raise capacity or world")
        r = min(ranks, key=lambda k: (load[k], used[k]))
        owner[f], load[r], used[r] = r, load[r] + traffic[f], used[r] + table_bytes[f]
    # refinement: move or swap between the most and the least loaded rank while the maximum drops
    for _ in range(4 * F):
        hi = max(range(world), key=load.__getitem__)
        lo = min(range(world), key=load.__getitem__)
        gap = load[hi] - load[lo]
        if gap <= 0:
            break
        best, best_gain = None, 0.0
        for f in (i for i in range(F) if owner[i] == hi):
            d = traffic[f]
            if 0 < d < gap and used[lo] + table_bytes[f] <= cap and min(d, gap - d) > best_gain:
                best, best_gain = (f, None), min(d, gap - d)
            for g in (i for i in range(F) if owner[i] == lo):
                d2 = traffic[f] - traffic[g]
                if 0 < d2 < gap and used[lo] - table_bytes[g] + table_bytes[f] <= cap \
                        and used[hi] - table_bytes[f] + table_bytes[g] <= cap and min(d2, gap - d2) > best_gain:
                    best, best_gain = (f, g), min(d2, gap - d2)
        if best is None:
            break
        f, g = best
        owner[f] = lo
        load[hi] -= traffic[f]
        load[lo] += traffic[f]
        used[hi] -= table_bytes[f]
        used[lo] += table_bytes[f]
        if g is not None:
            owner[g] = hi
            load[lo] -= traffic[g]
            load[hi] += traffic[g]
            used[lo] -= table_bytes[g]
            used[hi] += table_bytes[g]
    return owner


def _plan_two_loads(table_bytes, traffic, exchange, world: int, cap) -> List[int]:
    """plan_shards with two loads per table: minimise max over ranks of max(gather load, exchange load), each load
    expressed as a multiple of its per-rank mean."""
    F = len(table_bytes)
    na = sum(traffic) / world or 1.0
    nb = sum(exchange) / world or 1.0
    a = [t / na for t in traffic]
    b = [e / nb for e in exchange]
    owner = [-1] * F
    A, B, used = [0.0] * world, [0.0] * world, [0] * world
    for f in sorted(range(F), key=lambda i: (-max(a[i], b[i]), -table_bytes[i])):
        ranks = [r for r in range(world) if used[r] + table_bytes[f] <= cap]
        if not ranks:
            raise ValueError("tables do not fit the per-rank capacity with this greedy order; raise capacity or world")
        r = min(ranks, key=lambda k: (max(A[k] + a[f], B[k] + b[f]), A[k] + B[k], used[k]))
        owner[f] = r
        A[r] += a[f]
        B[r] += b[f]
        used[r] += table_bytes[f]
    peak = lambda r: max(A[r], B[r])
    for _ in range(4 * F):
        hi = max(range(world), key=peak)
        top = peak(hi)
        best, best_pair = None, top
        mine = [i for i in range(F) if owner[i] == hi]
        for r in range(world):
            if r == hi:
                continue
            theirs = [None] + [i for i in range(F) if owner[i] == r]
            for f in mine:
                for g in theirs:
                    ga, gb, gt = (a[g], b[g], table_bytes[g]) if g is not None else (0.0, 0.0, 0)
                    if used[r] + table_bytes[f] - gt > cap or used[hi] - table_bytes[f] + gt > cap:
                        continue
                    pair = max(A[hi] - a[f] + ga, B[hi] - b[f] + gb, A[r] + a[f] - ga, B[r] + b[f] - gb)
                    if pair < best_pair - 1e-12:
                        best, best_pair = (f, g, r), pair
        if best is None:
            break
        f, g, r = best
        owner[f] = r
        A[hi] -= a[f]; B[hi] -= b[f]; used[hi] -= table_bytes[f]
        A[r] += a[f]; B[r] += b[f]; used[r] += table_bytes[f]
        if g is not None:
            owner[g] = hi
            A[r] -= a[g]; B[r] -= b[g]; used[r] -= table_bytes[g]
            A[hi] += a[g]; B[hi] += b[g]; used[hi] += table_bytes[g]
    return owner


def shard_summary(owner: Sequence[int], table_bytes: Sequence[int], traffic: Sequence[float], world: int,
                  exchange: Optional[Sequence[float]] = None) -> dict:
    load = [0.0] * world
    used = [0] * world
    sent = [0.0] * world
    for f, r in enumerate(owner):
        load[r] += traffic[f]
        used[r] += table_bytes[f]
        if exchange is not None:
            sent[r] += exchange[f]
    mean = sum(load) / world if world else 0.0
    out = {"bytes_per_rank": used, "traffic_per_rank": load,
           "traffic_imbalance": (max(load) / mean) if mean > 0 else 1.0}
    if exchange is not None:
        mean_e = sum(sent) / world if world else 0.0
        out["exchange_per_rank"] = sent
        out["exchange_imbalance"] = (max(sent) / mean_e) if mean_e > 0 else 1.0
    return out


# ---------------------------------------------------------------------------
# sharded module
# ---------------------------------------------------------------------------
class ShardedFeatEmbed:
    """Table-wise sharded fused forward.

    owner[f]   rank that holds table f (from `plan_shards`); dims[f] = embedding dim of table f.
    local_tables  this rank's tables in increasing feature order (CUDA tensors), or None together with
               `pool_fn` for host-side tests.
    pool_fn    test hook only: `pool_fn(values, offsets, out)` must write the local features' pooled rows
               `[rows, sum(local dims)]` into `out`; the product path leaves it None and runs the CUDA
               library through `FeatEmbed`.  place_fn likewise (`place_fn(recv, out, rows)`).
    """

    def __init__(self, rank: int, world: int, owner: Sequence[int], dims: Sequence[int],
                 local_tables: Optional[List[torch.Tensor]] = None, device=None, group=None, chunks: int = 4,
                 pool_fn: Optional[Callable] = None, place_fn: Optional[Callable] = None, exchange: str = "nccl",
                 out_dtype: torch.dtype = torch.float32, columns: str = "owner", direct_hops: int = 0):
        if len(owner) != len(dims):
            raise ValueError("owner and dims must have one entry per feature")
        self.rank, self.world, self.group = rank, world, group
        self.owner, self.dims = list(owner), [int(d) for d in dims]
        self.chunks = max(1, int(chunks))
        self.local_features = [f for f, r in enumerate(self.owner) if r == rank]
        self.units = sum(self.dims)
        self.units_of = [sum(self.dims[f] for f, o in enumerate(self.owner) if o == r) for r in range(world)]
        self.local_units = self.units_of[rank]
        col, self.col_of = 0, []
        for d in self.dims:
            self.col_of.append(col)
            col += d
        self._pool_fn, self._place_fn = pool_fn, place_fn
        self.local = None
        if pool_fn is None:
            if local_tables is None or device is None:
                raise ValueError("the product path needs this rank's tables on a CUDA device (there is no CPU fallback)")
            from .rec_modules import FeatEmbed

            if len(local_tables) != len(self.local_features):
                raise ValueError(f"rank {rank} owns {len(self.local_features)} tables, got {len(local_tables)}")
            for t, f in zip(local_tables, self.local_features):
                if int(t.shape[1]) != self.dims[f]:
                    raise ValueError(f"table of feature {f} has dim {t.shape[1]}, expected {self.dims[f]}")
            self.device = torch.device(device)
            self.local = FeatEmbed(self.device, embed_tables=local_tables) if local_tables else None
            self._lib = _lib.load()
            self._comm = torch.cuda.Stream(device=self.device)
            self._copy_streams = [torch.cuda.Stream(device=self.device) for _ in range(min(4, max(1, world - 1)))]
        else:
            self.device = torch.device(device) if device is not None else torch.device("cpu")
        self._segs = {}      # rows per chunk -> device descriptor tensor for the placement kernel
        self._bufs = {}
        if exchange not in ("nccl", "peer", "copy", "push"):
            raise ValueError("exchange must be 'nccl', 'peer', 'copy' or 'push'")
        if exchange != "nccl" and pool_fn is not None:
            raise ValueError("the peer and copy exchanges exist only on GPUs")
        if out_dtype != torch.float32 and exchange == "nccl":
            raise ValueError("the NCCL exchange carries fp32 rows only")
        if columns not in ("owner", "canonical", "blocks"):
            raise ValueError("columns must be 'owner', 'canonical' or 'blocks'")
        if columns == "blocks" and exchange not in ("copy", "push"):
            raise ValueError("per-owner blocks are a result layout of the copy exchange")
        if columns == "canonical" and out_dtype != torch.float32:
            raise ValueError("the placement pass restores feature order for fp32 rows only")
        self.exchange, self.out_dtype, self.columns = exchange, out_dtype, columns
        if self.local is not None:
            self.local.set_output_dtype(out_dtype)
        # copy exchange: rank s's features side by side (increasing feature order) in one block, blocks in rank order
        self.block_col = [sum(self.units_of[:r]) for r in range(world)]
        nxt = list(self.block_col)
        self.owner_major_col = []
        for f, o in enumerate(self.owner):
            self.owner_major_col.append(nxt[o])
            nxt[o] += self.dims[f]
        # where feature f starts in a row of the result
        self.column_of = self.owner_major_col if (exchange in ("copy", "push") and columns != "canonical") else self.col_of
        if self.local is not None and exchange in ("copy", "push"):
            # hybrid: the nearest `direct_hops` destinations get their rows by kernel stores, the others by copies
            self.local.set_exchange_direct(int(direct_hops))
        if exchange == "push" and self.local is not None:
            self.local.set_exchange_engine("push")  # the copy exchange with SM copies instead of the copy engines
        self._copy_done = [None, None]
        self._peer = None    # (batch, own pointers, per-buffer pointer lists, output views, mapped peer pointers)
        self._step = 0

    # -- layout ------------------------------------------------------------
    def segments(self, rows: int) -> List[Tuple[int, int, int, int]]:
        """(src_off, src_ld, dst_col, width) of every feature inside a received chunk of `rows` samples:
        the chunk holds one block [rows, units_of[s]] per sender s, senders in rank order."""
        segs = []
        block = 0
        for s in range(self.world):
            c = 0
            for f, o in enumerate(self.owner):
                if o == s:
                    segs.append((block + c, self.units_of[s], self.col_of[f], self.dims[f]))
                    c += self.dims[f]
            block += rows * self.units_of[s]
        return segs

    def _segment_tensor(self, rows: int) -> torch.Tensor:
        t = self._segs.get(rows)
        if t is None:
            import numpy as np

            rec = np.zeros(len(self.dims), dtype=[("src_off", "<i8"), ("src_ld", "<i4"), ("dst_col", "<i4"),
                                                  ("width", "<i4"), ("pad", "<i4")])
            for i, (so, sl, dc, w) in enumerate(self.segments(rows)):
                rec[i] = (so, sl, dc, w, 0)
            t = torch.from_numpy(rec.view(np.uint8).copy()).to(self.device)
            self._segs[rows] = t
        return t

    # -- forward -----------------------------------------------------------
    def forward(self, values: Sequence[torch.Tensor], offsets: Sequence[torch.Tensor],
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """values/offsets: this rank's features (increasing feature order) for the WHOLE batch, offsets with
        batch + 1 entries.  Returns `[batch / world, sum(dim)]` fp32: this rank's samples, all features."""
        W, Cn = self.world, self.chunks
        if len(values) != len(self.local_features) or len(offsets) != len(self.local_features):
            raise ValueError(f"rank {self.rank} expects {len(self.local_features)} local features")
        if offsets:
            batch = offsets[0].numel() - 1
        else:
            batch = self._empty_rank_batch
        if self.exchange == "peer":
            return self._forward_peer(values, offsets, batch)
        if self.exchange in ("copy", "push"):
            return self._forward_copy(values, offsets, batch, out)
        if batch % (W * Cn) != 0:
            raise ValueError(f"batch {batch} must be a multiple of world * chunks = {W * Cn}")
        bc = batch // Cn          # samples per chunk
        rows = bc // W            # samples per chunk and rank
        key = (batch, str(self.device))
        bufs = self._bufs.get(key)
        if bufs is None:
            send = [torch.empty((bc, max(self.local_units, 1)), dtype=torch.float32, device=self.device)
                    for _ in range(min(Cn, 2))]
            recv = [torch.empty(rows * self.units, dtype=torch.float32, device=self.device) for _ in range(min(Cn, 2))]
            bufs = self._bufs[key] = (send, recv)
        send, recv = bufs
        if out is None:
            out = torch.empty((batch // W, self.units), dtype=torch.float32, device=self.device)
        in_split = [rows * self.local_units] * W
        out_split = [rows * self.units_of[s] for s in range(W)]
        cuda = self._pool_fn is None
        events = []
        for k in range(Cn):
            sb, rb = send[k % len(send)], recv[k % len(recv)]
            if cuda and k >= len(send):
                torch.cuda.current_stream(self.device).wait_event(events[k - len(send)])  # buffer reuse
            offs_k = [o[k * bc: (k + 1) * bc + 1] for o in offsets]
            if self.local_units:
                if cuda:
                    self.local(values, offs_k, out=sb)
                else:
                    self._pool_fn(values, offs_k, sb)
            out_k = out[k * rows: (k + 1) * rows]
            if cuda:
                ready = torch.cuda.Event()
                ready.record()
                with torch.cuda.stream(self._comm):
                    self._comm.wait_event(ready)
                    dist.all_to_all_single(rb, sb.view(-1)[: bc * self.local_units], out_split, in_split,
                                           group=self.group)
                    self._place(rb, out_k, rows)
                    done = torch.cuda.Event()
                    done.record()
                events.append(done)
            else:
                dist.all_to_all_single(rb, sb.reshape(-1)[: bc * self.local_units].contiguous(), out_split, in_split,
                                       group=self.group)
                self._place_fn(rb, out_k, rows)
        if cuda:
            torch.cuda.current_stream(self.device).wait_stream(self._comm)
        return out

    __call__ = forward

    # -- fused exchange over peer memory -------------------------------------
    def _setup_peer(self, batch: int):
        W = self.world
        if batch % W or (batch // W) % 32:
            raise ValueError(f"peer exchange needs batch / world to be a multiple of 32 (batch {batch}, world {W})")
        self._map_result_buffers(batch)
        if self.local is not None:
            self.local.set_output_columns([self.col_of[f] for f in self.local_features], self.units)

    def _map_result_buffers(self, batch: int):
        """Two result matrices [batch / world, units] per rank, allocated by the library and mapped into every
        other rank's process (CUDA IPC)."""
        W = self.world
        rows = batch // W
        es = 4 if self.out_dtype == torch.float32 else 2
        nbytes = rows * self.units * es
        own, handles = [], torch.empty((2, 64), dtype=torch.uint8)
        for b in range(2):
            ptr = C.c_void_p()
            hbuf = (C.c_ubyte * 64)()
            _lib.check(self._lib.eb_peer_alloc(self.device.index, nbytes, C.byref(ptr), hbuf))
            own.append(int(ptr.value))
            handles[b] = torch.tensor(list(hbuf), dtype=torch.uint8)
        gathered = [torch.empty((2, 64), dtype=torch.uint8, device=self.device) for _ in range(W)]
        dist.all_gather(gathered, handles.to(self.device), group=self.group)
        ptrs, mapped = [[0] * W for _ in range(2)], []
        for r in range(W):
            hs = gathered[r].cpu()
            for b in range(2):
                if r == self.rank:
                    ptrs[b][r] = own[b]
                else:
                    raw = (C.c_ubyte * 64)(*hs[b].tolist())
                    p = C.c_void_p()
                    _lib.check(self._lib.eb_peer_open(self.device.index, raw, C.byref(p)))
                    ptrs[b][r] = int(p.value)
                    mapped.append(int(p.value))

        units = self.units
        typestr = "<f4" if es == 4 else "<i2"

        class _View:  # torch view of a library-owned buffer
            def __init__(self, ptr):
                self.__cuda_array_interface__ = {"shape": (rows, units), "typestr": typestr, "data": (ptr, False),
                                                 "version": 2}

        views = [torch.as_tensor(_View(p), device=self.device) for p in own]
        if es == 2:
            views = [v.view(self.out_dtype) for v in views]
        self._flag = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._peer = (batch, own, ptrs, views, mapped)

    # -- exchange through the copy engines -------------------------------------
    def _forward_copy(self, values, offsets, batch: int, out: Optional[torch.Tensor]) -> torch.Tensor:
        W, Cn = self.world, self.chunks
        if batch % (W * Cn) != 0:
            raise ValueError(f"batch {batch} must be a multiple of world * chunks = {W * Cn}")
        if self._peer is None or self._peer[0] != batch:
            self.close()
            self._map_result_buffers(batch)
            self._send = [torch.empty((batch, max(self.local_units, 1)), dtype=self.out_dtype, device=self.device)
                          for _ in range(2)] if self.local is not None else None
            self._copy_done = [None, None]
        _, _, ptrs, views, _ = self._peer
        b = self._step % 2
        self._step += 1
        cur = torch.cuda.current_stream(self.device)
        if self._copy_done[b] is not None:
            cur.wait_event(self._copy_done[b])  # the copies that read this send buffer two calls ago are done
        rows = batch // W
        es = 4 if self.out_dtype == torch.float32 else 2
        blocked = self.columns != "owner"
        if self.local is not None:
            if blocked:
                # the result buffer holds one contiguous block [rows, units of rank s] per owner rank s: every copy is
                # one contiguous run on both sides
                mine = rows * self.block_col[self.rank] * es
                self.local.forward_exchange(values, offsets, self._send[b], [p + mine for p in ptrs[b]], self.rank,
                                            self.local_units, 0, Cn, self._copy_streams)
            else:
                self.local.forward_exchange(values, offsets, self._send[b], ptrs[b], self.rank, self.units,
                                            self.block_col[self.rank], Cn, self._copy_streams)
        with torch.cuda.stream(self._comm):
            self._comm.wait_stream(cur)  # the kernel stores this rank's own samples itself
            for cs in self._copy_streams:
                self._comm.wait_stream(cs)
            dist.all_reduce(self._flag, group=self.group)  # after it, every rank's copies into my matrix are complete
            done = torch.cuda.Event()
            done.record()
        self._copy_done[b] = done
        cur.wait_stream(self._comm)
        if self.columns == "owner":
            return views[b]
        flat = views[b].view(-1)
        if self.columns == "blocks":
            return [flat[rows * self.block_col[s2]: rows * (self.block_col[s2] + self.units_of[s2])].view(rows, self.units_of[s2])
                    for s2 in range(W)]
        if out is None:
            out = torch.empty((rows, self.units), dtype=torch.float32, device=self.device)
        self._place(flat, out, rows)  # blocks -> feature order
        return out

    def _forward_peer(self, values, offsets, batch: int) -> torch.Tensor:
        if self._peer is None or self._peer[0] != batch:
            self.close()
            self._setup_peer(batch)
        _, _, ptrs, views, _ = self._peer
        b = self._step % 2
        self._step += 1
        if self.local is not None:
            self.local.forward_peers(values, offsets, ptrs[b], self.units)
        dist.all_reduce(self._flag, group=self.group)  # every rank's stores into my buffer are complete after this
        return views[b]

    def close(self) -> None:
        """Unmap peers' buffers and free this rank's (call on every rank, after a barrier).  Tensors returned by
        the peer and copy exchanges are views of these buffers and are invalid from here on."""
        if self._peer is not None:
            _, own, _, views, mapped = self._peer
            del views
            torch.cuda.synchronize(self.device)
            for p in mapped:
                self._lib.eb_peer_close(self.device.index, C.c_void_p(p))
            dist.barrier(group=self.group)  # nobody still maps my buffers when I free them
            for p in own:
                self._lib.eb_peer_free(self.device.index, C.c_void_p(p))
            self._peer = None

    _empty_rank_batch = 0

    def set_batch_for_empty_rank(self, batch: int) -> None:
        """A rank that owns no table cannot read the batch size from its inputs; tell it."""
        self._empty_rank_batch = int(batch)

    def _place(self, recv: torch.Tensor, out_k: torch.Tensor, rows: int) -> None:
        segs = self._segment_tensor(rows)
        _lib.check(self._lib.eb_place_columns(C.c_void_p(recv.data_ptr()), C.c_void_p(out_k.data_ptr()), rows,
                                              out_k.stride(0), len(self.dims), C.c_void_p(segs.data_ptr()),
                                              self.device.index,
                                              C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)))


def local_sample_ids(batch: int, world: int, chunks: int, rank: int) -> List[int]:
    """Batch positions of the samples rank `rank` ends up with, in its output row order."""
    bc = batch // chunks
    rows = bc // world
    return [k * bc + rank * rows + j for k in range(chunks) for j in range(rows)]
