"""PyTorch modules with the interface of RecFlex's `RecFlex/rec_modules.py`.

`FeatEmbed` owns the embedding tables and runs the fused multi-feature
embedding-bag forward (sum pooling, outputs of all features concatenated into
one `[batch, sum(dim_f)]` fp32 tensor) through the C ABI of
librecflex_b200.so.  `FeatPreprocess` turns the reference's text input (one
string of comma-separated indices per sample and feature) into per-feature
`values` / `offsets` tensors, and `FeatProcessEmbed` composes the two exactly
like the reference's class of the same name (rec_modules.py:114-140).

PyTorch is used for device memory, streams and module plumbing only; there is
no PyTorch or CPU implementation of the forward behind these classes.
"""
from __future__ import annotations

import ctypes as C
from concurrent.futures import ThreadPoolExecutor
from types import ModuleType
from typing import List, Optional, Sequence, Tuple, Union

import numpy as np
import torch
import torch.nn as nn

from . import _lib
from ._lib import EbSchedule


def _device_index(device) -> int:
    dev = torch.device(device) if not isinstance(device, int) else torch.device("cuda", device)
    if dev.type != "cuda":
        raise ValueError(f"FeatEmbed needs a CUDA device, got {dev}")
    return dev.index if dev.index is not None else torch.cuda.current_device()


class Schedule:
    """One feature's schedule: kind ('auto' | 'group' | 'warp' | 'flat' | 'stream' | 'pipe'), unroll, bags_per_tile.

    The counterpart of the reference's (ScheduleBase subclass, params NamedTuple)
    pair (code_emitter/schedule_base.py:54-87); see include/recflex_b200.h for
    what each kind does.
    """

    __slots__ = ("kind", "unroll", "bags_per_tile")

    def __init__(self, kind: Union[str, int] = "auto", unroll: int = 0, bags_per_tile: int = 0):
        self.kind = _lib.SCHED_KINDS[kind] if isinstance(kind, str) else int(kind)
        self.unroll = int(unroll)
        self.bags_per_tile = int(bags_per_tile)

    def to_c(self) -> EbSchedule:
        return EbSchedule(self.kind, self.unroll, 0, self.bags_per_tile)

    def to_json(self) -> dict:
        return {"kind": _lib.SCHED_NAMES[self.kind], "unroll": self.unroll, "bags_per_tile": self.bags_per_tile}

    @staticmethod
    def from_json(d: dict) -> "Schedule":
        return Schedule(d["kind"], d.get("unroll", 0), d.get("bags_per_tile", 0))

    def __repr__(self) -> str:
        return f"Schedule({_lib.SCHED_NAMES[self.kind]!r}, unroll={self.unroll}, bags_per_tile={self.bags_per_tile})"

    def __eq__(self, other) -> bool:
        return isinstance(other, Schedule) and (self.kind, self.unroll, self.bags_per_tile) == (
            other.kind, other.unroll, other.bags_per_tile)


class FeatEmbed(nn.Module):
    """Fused embedding-bag forward over a list of tables (rec_modules.py:57-111 in the reference).

    Parameters mirror the reference: either `embed_tables` (a list of
    `[rows, dim]` CUDA tensors, fp32 or fp16, which the module keeps alive and
    whose storage must not move) or `table_shapes` (a list of `(rows, dim)`;
    tables are then created with `torch.randn` in `dtype`).
    """

    def __init__(self, device, embed_tables: Optional[List[torch.Tensor]] = None,
                 table_shapes: Optional[Sequence[Tuple[int, int]]] = None, dtype: torch.dtype = torch.float32):
        super().__init__()
        self._h = C.c_void_p()
        self._lib = _lib.load()  # raises when the CUDA library is missing: there is no fallback
        self.device = torch.device("cuda", _device_index(device))
        if embed_tables:
            self.embed_tables = list(embed_tables)
        elif table_shapes:
            self.embed_tables = [torch.randn(tuple(s), dtype=dtype, device=self.device) for s in table_shapes]
        else:
            raise Exception("At least one of embed_tables and table_shapes should be given!")
        F = len(self.embed_tables)
        rows = (C.c_int64 * F)()
        dims = (C.c_int32 * F)()
        dtypes = (C.c_int32 * F)()
        ptrs = (C.c_void_p * F)()
        for f, t in enumerate(self.embed_tables):
            if t.dim() != 2 or not t.is_cuda or t.device != self.device or not t.is_contiguous():
                raise ValueError(f"table {f} must be a contiguous 2-D tensor on {self.device}")
            if t.dtype not in (torch.float32, torch.float16):
                raise ValueError(f"table {f}: dtype {t.dtype} is not supported (float32 or float16)")
            rows[f], dims[f] = t.shape[0], t.shape[1]
            dtypes[f] = _lib.EB_F32 if t.dtype == torch.float32 else _lib.EB_F16
            ptrs[f] = t.data_ptr()
        _lib.check(self._lib.eb_create(C.byref(self._h), self.device.index, F, rows, dims, dtypes, ptrs))
        # raw device pointers, as the reference keeps them (rec_modules.py:70)
        self.embed_table_ptrs = torch.tensor([t.data_ptr() for t in self.embed_tables], dtype=torch.int64)
        self.num_features = F
        self.output_units = sum(int(t.shape[1]) for t in self.embed_tables)
        ws = C.c_size_t()
        _lib.check(self._lib.eb_workspace_bytes(self._h, C.byref(ws)))
        self._ws_bytes = int(ws.value)
        self._ws = torch.zeros(self._ws_bytes + 128, dtype=torch.uint8, device=self.device)  # chunk flags start at 0
        self._ws_ptr = (self._ws.data_ptr() + 127) // 128 * 128
        self._staging = None
        self._staging_ptr = 0
        self._staging_bytes = 0
        self.output_dtype = torch.float32

    def __del__(self):
        # may run while the interpreter shuts down, when nn.Module's attribute machinery is already gone
        try:
            h = self.__dict__.get("_h")
            if h is not None and h.value:
                self.__dict__["_h"] = None
                self._lib.eb_destroy(h)
        except Exception:
            pass

    # -- schedules ---------------------------------------------------------
    @property
    def max_concurrent_blocks(self) -> int:
        """Persistent CTAs of the fused kernel (reference: torch.ops.recom.get_max_concurrent_blocks)."""
        n = C.c_int()
        _lib.check(self._lib.eb_max_concurrent_ctas(self._h, 0, C.byref(n)))
        return int(n.value)

    def set_schedules(self, schedules: Optional[Sequence[Schedule]] = None, occupancy: int = 0) -> None:
        arr = None
        if schedules is not None:
            if len(schedules) != self.num_features:
                raise ValueError(f"{len(schedules)} schedules for {self.num_features} features")
            arr = (EbSchedule * self.num_features)(*[s.to_c() for s in schedules])
        _lib.check(self._lib.eb_set_schedules(self._h, arr, int(occupancy)))

    def get_schedules(self) -> Tuple[List[Schedule], int]:
        arr = (EbSchedule * self.num_features)()
        occ = C.c_int()
        _lib.check(self._lib.eb_get_schedules(self._h, arr, C.byref(occ)))
        return [Schedule(s.kind, s.unroll, s.bags_per_tile) for s in arr], int(occ.value)

    _OUT_DTYPES = {torch.float32: _lib.EB_OUT_F32, torch.bfloat16: _lib.EB_OUT_BF16, torch.float16: _lib.EB_OUT_F16}

    def set_output_dtype(self, dtype: torch.dtype) -> None:
        """Element type of the pooled output: torch.float32 (default, the reference's contract), or torch.bfloat16 /
        torch.float16 for consumers that cast anyway (sums are still accumulated in fp32 and rounded once on the
        way out).  Output tensors passed as `out=` must then have this dtype."""
        if dtype not in self._OUT_DTYPES:
            raise TypeError(f"output dtype must be float32, bfloat16 or float16, got {dtype}")
        _lib.check(self._lib.eb_set_output_dtype(self._h, self._OUT_DTYPES[dtype]))
        self.output_dtype = dtype

    def set_long_bag_split(self, min_bytes: int) -> None:
        """Bags whose rows add up to `min_bytes` or more (default 1 MB) are pooled by many warps in a second kernel
        instead of by the one warp that meets them; 0 pools every bag in place."""
        _lib.check(self._lib.eb_set_long_bag_split(self._h, int(min_bytes)))

    def set_exchange_engine(self, engine: str) -> None:
        """Who ships the finished pieces of `forward_exchange`: 'copy' (the copy engines, default) or 'push' (a small
        kernel whose warps store 512-byte runs to the peers)."""
        code = {"copy": _lib.EB_EXCHANGE_COPY_ENGINES, "push": _lib.EB_EXCHANGE_SM_PUSH}[engine]
        _lib.check(self._lib.eb_set_exchange_engine(self._h, code))

    def set_exchange_direct(self, hops: int) -> None:
        """`forward_exchange`: the rows for the `hops` ranks to the right of this one are stored by the kernel
        straight into their result blocks; only the other destinations go through the send buffer and the copies."""
        _lib.check(self._lib.eb_set_exchange_direct(self._h, int(hops)))

    def _check_out(self, out: Optional[torch.Tensor], batch: int) -> torch.Tensor:
        if out is None:
            return torch.empty((batch, self.output_units), dtype=self.output_dtype, device=self.device)
        if out.dtype != self.output_dtype or out.dim() != 2 or out.shape[0] != batch or out.stride(1) != 1 \
                or out.shape[1] < self.output_units:
            raise ValueError(f"out must be a {self.output_dtype} [batch, >= output_units] tensor with unit column stride")
        return out

    # -- forward -----------------------------------------------------------
    def _stream(self) -> C.c_void_p:
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    @staticmethod
    def _index_dtype(t: torch.Tensor) -> int:
        if t.dtype == torch.int32:
            return _lib.EB_I32
        if t.dtype == torch.int64:
            return _lib.EB_I64
        raise TypeError(f"values/offsets must be int32 or int64, got {t.dtype}")

    def forward(self, values: Sequence[torch.Tensor], offsets: Sequence[torch.Tensor],
                include_last_offset: bool = True, timing: bool = False, timing_schedules: Optional[int] = None,
                out: Optional[torch.Tensor] = None):
        """Pool every feature's bags and concatenate: returns fp32 `[batch, output_units]`.

        values[f]: 1-D int32/int64 indices into table f; offsets[f]: bag starts,
        `batch + 1` entries ending with `len(values[f])` (the reference's device
        format) or `batch` entries with `include_last_offset=False` (the
        torch.nn.EmbeddingBag default).  With `timing=True` returns
        `(output, per_feature_times)` like the reference (rec_modules.py:96-109):
        a float64 tensor of summed per-tile device time in milliseconds for the
        first `timing_schedules` features.
        """
        F = self.num_features
        if len(values) != F or len(offsets) != F:
            raise ValueError(f"expected {F} values and offsets tensors, got {len(values)} and {len(offsets)}")
        idt = self._index_dtype(values[0])
        n_off = offsets[0].numel()
        batch = n_off - 1 if include_last_offset else n_off
        if batch < 0:
            raise ValueError("offsets with include_last_offset=True need at least one entry")
        vp = (C.c_void_p * F)()
        op = (C.c_void_p * F)()
        nnz = (C.c_int64 * F)()
        keep = []
        for f in range(F):
            v, o = values[f], offsets[f]
            if self._index_dtype(v) != idt or self._index_dtype(o) != idt:
                raise TypeError("all values and offsets tensors must share one integer dtype")
            if o.numel() != n_off:
                raise ValueError(f"feature {f}: offsets has {o.numel()} entries, feature 0 has {n_off}")
            if v.device != self.device or o.device != self.device:
                raise ValueError(f"feature {f}: values/offsets must live on {self.device}")
            if not v.is_contiguous():
                v = v.contiguous()
            if not o.is_contiguous():
                o = o.contiguous()
            keep.append((v, o))
            vp[f], op[f], nnz[f] = v.data_ptr(), o.data_ptr(), v.numel()
        out = self._check_out(out, batch)
        ld = out.stride(0) if batch > 1 else max(out.shape[1], self.output_units)
        if not timing:
            _lib.check(self._lib.eb_forward(self._h, batch, vp, op, nnz, idt, int(include_last_offset),
                                            C.c_void_p(out.data_ptr()), ld, C.c_void_p(self._ws_ptr),
                                            self._ws_bytes, self._stream()))
            return out
        ns = (C.c_double * F)()
        _lib.check(self._lib.eb_forward_timed(self._h, batch, vp, op, nnz, idt, int(include_last_offset),
                                              C.c_void_p(out.data_ptr()), ld, C.c_void_p(self._ws_ptr),
                                              self._ws_bytes, self._stream(), ns))
        n_t = F if not timing_schedules or timing_schedules > F else timing_schedules
        times = torch.tensor([ns[f] * 1e-6 for f in range(n_t)], dtype=torch.float64)
        return out, times

    def set_output_columns(self, first_column: Optional[Sequence[int]], units: int = 0) -> None:
        """Feature f writes columns [first_column[f], first_column[f] + dim_f) of a `units`-wide output row
        (None restores the default side-by-side layout)."""
        if first_column is None:
            _lib.check(self._lib.eb_set_output_columns(self._h, None, 0))
            self.output_units = sum(int(t.shape[1]) for t in self.embed_tables)
            return
        if len(first_column) != self.num_features:
            raise ValueError(f"{len(first_column)} columns for {self.num_features} features")
        arr = (C.c_int32 * self.num_features)(*[int(c) for c in first_column])
        _lib.check(self._lib.eb_set_output_columns(self._h, arr, int(units)))
        self.output_units = int(units)

    def set_kernel_overlap(self, fused_ctas_per_sm: int) -> None:
        """n > 0: the fused kernel runs on n CTAs per SM and the warp-per-bag kernel beside it on a stream of the
        handle (joined back into the current stream); 0: one after the other on the current stream (default)."""
        _lib.check(self._lib.eb_set_kernel_overlap(self._h, int(fused_ctas_per_sm)))

    def set_peer_interleave(self, enabled: bool) -> None:
        """forward_peers deals a feature's consecutive tiles round-robin over the destination ranks (default) or
        walks the batch in order (False).  Same results; only the NVLink traffic pattern changes."""
        _lib.check(self._lib.eb_set_peer_interleave(self._h, 1 if enabled else 0))

    def forward_peers(self, values: Sequence[torch.Tensor], offsets: Sequence[torch.Tensor],
                      peer_ptrs: Sequence[int], out_ld: int) -> None:
        """Fused pooling + exchange: sample b goes to the output matrix of rank b // (batch / world) whose
        device pointer (as seen from this process) is peer_ptrs[rank].  offsets carry batch + 1 entries."""
        F, W = self.num_features, len(peer_ptrs)
        idt = self._index_dtype(values[0])
        batch = offsets[0].numel() - 1
        vp = (C.c_void_p * F)()
        op = (C.c_void_p * F)()
        nnz = (C.c_int64 * F)()
        for f in range(F):
            v, o = values[f], offsets[f]
            if self._index_dtype(v) != idt or self._index_dtype(o) != idt:
                raise TypeError("all values and offsets tensors must share one integer dtype")
            if o.numel() != batch + 1 or not v.is_contiguous() or not o.is_contiguous():
                raise ValueError(f"feature {f}: offsets need batch + 1 entries; tensors must be contiguous")
            if v.device != self.device or o.device != self.device:
                raise ValueError(f"feature {f}: values/offsets must live on {self.device}")
            vp[f], op[f], nnz[f] = v.data_ptr(), o.data_ptr(), v.numel()
        pp = (C.c_void_p * W)(*[int(p) for p in peer_ptrs])
        _lib.check(self._lib.eb_forward_peers(self._h, batch, vp, op, nnz, idt, 1, pp, W, int(out_ld),
                                              C.c_void_p(self._ws_ptr), self._ws_bytes, self._stream()))

    def _feature_pointers(self, values, offsets):
        F = self.num_features
        idt = self._index_dtype(values[0])
        batch = offsets[0].numel() - 1
        vp = (C.c_void_p * F)()
        op = (C.c_void_p * F)()
        nnz = (C.c_int64 * F)()
        for f in range(F):
            v, o = values[f], offsets[f]
            if self._index_dtype(v) != idt or self._index_dtype(o) != idt:
                raise TypeError("all values and offsets tensors must share one integer dtype")
            if o.numel() != batch + 1 or not v.is_contiguous() or not o.is_contiguous():
                raise ValueError(f"feature {f}: offsets need batch + 1 entries; tensors must be contiguous")
            if v.device != self.device or o.device != self.device:
                raise ValueError(f"feature {f}: values/offsets must live on {self.device}")
            vp[f], op[f], nnz[f] = v.data_ptr(), o.data_ptr(), v.numel()
        return idt, batch, vp, op, nnz

    def forward_exchange(self, values: Sequence[torch.Tensor], offsets: Sequence[torch.Tensor], send: torch.Tensor,
                         peer_ptrs: Sequence[int], rank: int, out_ld: int, out_col: int, chunks: int,
                         copy_streams: Sequence[torch.cuda.Stream]) -> None:
        """Pooling + copy-engine exchange (see eb_forward_exchange in include/recflex_b200.h): pools the whole batch
        into `send` ([batch, >= output_units], this module's output dtype) piece by piece and lets `copy_streams`
        ship every finished piece to the other ranks' matrices `peer_ptrs` at columns [out_col, out_col +
        output_units); this rank's own samples are stored straight into peer_ptrs[rank] by the kernel."""
        idt, batch, vp, op, nnz = self._feature_pointers(values, offsets)
        send = self._check_out(send, batch)
        W = len(peer_ptrs)
        pp = (C.c_void_p * W)(*[int(p) for p in peer_ptrs])
        _lib.check(self._lib.eb_forward_exchange(self._h, batch, vp, op, nnz, idt, 1, C.c_void_p(send.data_ptr()),
                                                 send.stride(0), pp, W, int(rank), int(out_ld), int(out_col),
                                                 int(chunks), C.c_void_p(self._ws_ptr), self._ws_bytes, self._stream(),
                                                 (C.c_void_p * len(copy_streams))(*[s.cuda_stream for s in copy_streams]),
                                                 len(copy_streams)))

    def forward_packed(self, values: torch.Tensor, offsets: torch.Tensor, out: Optional[torch.Tensor] = None):
        """Same forward for one packed batch: `values` = all features' indices back to back,
        `offsets` = `[num_features, batch + 1]`, both on the device."""
        if offsets.dim() != 2 or offsets.shape[0] != self.num_features or not offsets.is_contiguous():
            raise ValueError("offsets must be a contiguous [num_features, batch + 1] tensor")
        idt = self._index_dtype(values)
        if self._index_dtype(offsets) != idt:
            raise TypeError("values and offsets must share one integer dtype")
        batch = offsets.shape[1] - 1
        out = self._check_out(out, batch)
        ld = out.stride(0) if batch > 1 else max(out.shape[1], self.output_units)
        _lib.check(self._lib.eb_forward_packed(self._h, batch, C.c_void_p(values.data_ptr()),
                                               C.c_void_p(offsets.data_ptr()), idt, C.c_void_p(out.data_ptr()), ld,
                                               C.c_void_p(self._ws_ptr), self._ws_bytes, self._stream()))
        return out

    def offsets_from_lengths(self, lengths: torch.Tensor) -> torch.Tensor:
        """Device tensor `[num_features, batch]` of bag lengths -> `[num_features, batch + 1]` offsets for
        `forward_packed` (computed on the device, no host pass)."""
        if lengths.dim() != 2 or lengths.shape[0] != self.num_features or not lengths.is_contiguous():
            raise ValueError("lengths must be a contiguous [num_features, batch] tensor")
        if lengths.device != self.device:
            raise ValueError(f"lengths must live on {self.device}")
        idt = self._index_dtype(lengths)
        offsets = torch.empty((self.num_features, lengths.shape[1] + 1), dtype=lengths.dtype, device=self.device)
        _lib.check(self._lib.eb_offsets_from_lengths(C.c_void_p(lengths.data_ptr()), C.c_void_p(offsets.data_ptr()),
                                                     self.num_features, lengths.shape[1], idt, self.device.index,
                                                     self._stream()))
        return offsets

    def forward_host(self, values: torch.Tensor, offsets: torch.Tensor, out: Optional[torch.Tensor] = None):
        """End-to-end call on HOST tensors (pinned for full copy speed): uploads the packed batch,
        runs the forward and downloads the `[batch, output_units]` result into `out` (a host
        tensor, allocated pinned when omitted).  Returns after enqueueing on the current stream."""
        if values.is_cuda or offsets.is_cuda:
            raise ValueError("forward_host takes host tensors")
        idt = self._index_dtype(values)
        batch = offsets.shape[1] - 1
        if out is None:
            out = torch.empty((batch, self.output_units), dtype=self.output_dtype, pin_memory=True)
        elif out.dtype != self.output_dtype or out.is_cuda or not out.is_contiguous() \
                or out.numel() != batch * self.output_units:
            raise ValueError(f"out must be a contiguous host {self.output_dtype} [batch, output_units] tensor")
        need = C.c_size_t()
        _lib.check(self._lib.eb_host_staging_bytes(self._h, batch, values.numel(), idt, C.byref(need)))
        if self._staging_bytes < need.value:
            self._staging = torch.empty(int(need.value) + 256, dtype=torch.uint8, device=self.device)
            self._staging_ptr = (self._staging.data_ptr() + 255) // 256 * 256
            self._staging_bytes = int(need.value)
        _lib.check(self._lib.eb_forward_host(self._h, batch, C.c_void_p(values.data_ptr()), values.numel(),
                                             C.c_void_p(offsets.data_ptr()), idt, C.c_void_p(out.data_ptr()),
                                             C.c_void_p(self._staging_ptr), self._staging_bytes,
                                             C.c_void_p(self._ws_ptr), self._ws_bytes, self._stream()))
        return out

    def kernel_timing(self, enable: bool = True) -> None:
        """Record a CUDA event pair around every fused-kernel launch from now on (ring of 256)."""
        _lib.check(self._lib.eb_kernel_timing(self._h, int(enable)))

    def kernel_times(self) -> List[float]:
        """Milliseconds of each fused-kernel launch since the last read (synchronises on them)."""
        buf = (C.c_float * 256)()
        n = C.c_int()
        _lib.check(self._lib.eb_kernel_times(self._h, buf, 256, C.byref(n)))
        return [float(buf[i]) for i in range(n.value)]

    def last_binding(self) -> List[int]:
        """Bags per warp tile the device chose for every feature in the last forward (synchronises)."""
        arr = (C.c_int32 * self.num_features)()
        _lib.check(self._lib.eb_last_binding(self._h, C.c_void_p(self._ws_ptr), self._stream(), arr))
        return [int(x) for x in arr]

    def check_status(self) -> None:
        """Raise if the last forward met an out-of-range index or non-monotone offsets (synchronises)."""
        _lib.check(self._lib.eb_check_status(self._h, C.c_void_p(self._ws_ptr), self._stream()))


def parse_bags(lines: Sequence[str]) -> Tuple[np.ndarray, np.ndarray]:
    """One feature's text batch -> (values int32, offsets int32 [batch + 1]) with the reference's
    parsing rules (examples/csrc/warp_per_sample_preprocess.cu:6-38): every non-digit character
    ends a number, an empty string is an empty bag."""
    lib = _lib.load()
    text = "\n".join(lines).encode()
    batch = len(lines)
    cap = len(text) + 1
    values = np.empty(cap, dtype=np.int32)
    offsets = np.empty(batch + 1, dtype=np.int32)
    nnz = C.c_int64()
    _lib.check(lib.eb_parse_bags(text, len(text), batch, values.ctypes.data_as(C.c_void_p), cap,
                                 offsets.ctypes.data_as(C.c_void_p), C.byref(nnz)))
    return values[: nnz.value].copy(), offsets


class FeatPreprocess(nn.Module):
    """Text batch -> device tensors (reference: rec_modules.py:19-54).

    `recom_host` is accepted for signature compatibility and ignored: the
    parser lives in librecflex_b200.so and tiling / block binding happen on the
    device inside the forward.
    """

    def __init__(self, recom_host: Optional[ModuleType], device):
        super().__init__()
        self.recom_host = recom_host
        self.device = torch.device("cuda", _device_index(device))
        self._pool = ThreadPoolExecutor(max_workers=8)

    def forward(self, raw_data: List[List[str]], max_concurrent_blocks: int = 0):
        parsed = list(self._pool.map(parse_bags, raw_data))  # ctypes releases the GIL: features parse in parallel
        values = [torch.from_numpy(v).to(self.device, non_blocking=True) for v, _ in parsed]
        offsets = [torch.from_numpy(o).to(self.device, non_blocking=True) for _, o in parsed]
        return values, offsets


class FeatProcessEmbed(nn.Module):
    """Preprocess + embed (reference: rec_modules.py:114-140), same constructor and forward arguments."""

    def __init__(self, recom_host: Optional[ModuleType] = None, device=None,
                 embed_tables: Optional[List[torch.Tensor]] = None,
                 table_shapes: Optional[Sequence[Tuple[int, int]]] = None, librecom_path: Optional[str] = None):
        super().__init__()
        if device is None:
            device = torch.cuda.current_device()
        self.device = torch.device("cuda", _device_index(device))
        self.preprocess_layer = FeatPreprocess(recom_host, device=self.device)
        self.embed_layer = FeatEmbed(device=self.device, embed_tables=embed_tables, table_shapes=table_shapes)
        self.max_concurrent_blocks = self.embed_layer.max_concurrent_blocks

    def forward(self, raw_data: List[List[str]], timing: bool = False, timing_schedules: Optional[int] = None,
                timing_kernel: bool = False):
        values, offsets = self.preprocess_layer(raw_data, self.max_concurrent_blocks)
        if not timing_kernel:
            return self.embed_layer(values, offsets, timing=timing, timing_schedules=timing_schedules)
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        result = self.embed_layer(values, offsets, timing=timing, timing_schedules=timing_schedules)
        end.record()
        end.synchronize()
        return result, start.elapsed_time(end)


class RecomModel(nn.Module):
    """Fused embedding + MLP (reference: rec_modules.py:143-179): embed -> [batch, output_units] -> MLP -> sigmoid.

    `mlp_dtype` (not in the reference, whose model is fp32 throughout) selects the MLP's precision.  With
    torch.bfloat16 or torch.float16 the embedding layer writes its pooled sums directly in that type
    (`FeatEmbed.set_output_dtype`), i.e. in the first linear layer's input layout and dtype: no fp32 intermediate is
    written or re-read, and the cast costs nothing."""

    def __init__(self, mlp_unit_nums: List[int], device, embed_tables: Optional[List[torch.Tensor]] = None,
                 table_shapes: Optional[Sequence[Tuple[int, int]]] = None, mlp_dtype: torch.dtype = torch.float32):
        super().__init__()
        self.device = torch.device("cuda", _device_index(device))
        self.embed_layer = FeatEmbed(device=self.device, embed_tables=embed_tables, table_shapes=table_shapes)
        self.embed_layer.set_output_dtype(mlp_dtype)
        layers = []
        unit_nums = [self.embed_layer.output_units] + list(mlp_unit_nums) + [1]
        for i in range(len(unit_nums) - 1):
            layers.append(nn.Linear(unit_nums[i], unit_nums[i + 1], bias=True, device=self.device, dtype=mlp_dtype))
            layers.append(nn.Sigmoid() if i + 2 == len(unit_nums) else nn.ReLU())
        self.mlp = nn.Sequential(*layers)

    def forward(self, values: Sequence[torch.Tensor], offsets: Sequence[torch.Tensor],
                include_last_offset: bool = True):
        embed_output = self.embed_layer(values, offsets, include_last_offset=include_last_offset)
        return self.mlp(embed_output)
