"""Tensor parallelism with the collectives fused into the GEMM kernels (F3 / F4).

Megatron-style sharding with sequence-parallel regions: activations between TP layers hold ``T / tp`` tokens per
rank; ``ColumnParallelLinear`` (in_proj / QKV / gate-up) is all-gather -> GEMM, ``RowParallelLinear``
(out_proj / o_proj / down) is GEMM -> reduce-scatter. On CUDA the collective runs inside ``sx_gemm_bf16_comm``
over symmetric memory; with ``fused=False`` (and on CPU/gloo) the same layers call ``torch.distributed``
collectives around the plain GEMM, which is the baseline the fused kernels are measured against.
The reference's ``sneppx_tp_linear_forward`` / ``sneppx_tp_all_reduce`` run one local cublasSgemm and copy
(kernel/distributed/tensor_parallel.c:58-108).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist
import torch.nn as tnn

from ..nn.modules import Module
from ..ops import _lib
from ..ops.gemm import gemm
from .symm import SxPeers

AG_SIG, AG_DONE, RS_DONE = 8, 9, 10
RS_COUNTER_WORD0 = 16 * 16  # channels 16..47 of the pad hold reduce-scatter row-block counters


class SxGemmCommArgs(C.Structure):
    _fields_ = [("peers", SxPeers), ("mode", C.c_int), ("flags", C.c_void_p), ("epoch", C.c_uint), ("n_copy", C.c_int),
                ("chunk_rows", C.c_int), ("sub_rows", C.c_int), ("sig_channel", C.c_int), ("done_channel", C.c_int),
                ("counter_word", C.c_int), ("rs_expected", C.c_uint), ("rs_out", C.c_void_p),
                ("rs_residual", C.c_void_p), ("rs_ldd", C.c_longlong), ("cta_counter", C.c_void_p),
                ("ep_x", C.c_void_p), ("ep_dest_rank", C.c_void_p), ("ep_dest_row", C.c_void_p),
                ("ep_row_scale", C.c_void_p), ("ep_entries", C.c_int), ("ep_k", C.c_int), ("ep_d", C.c_int),
                ("ep_arrive", C.c_void_p * 8), ("ep_tile_expected", C.c_void_p)]


def _gemm_args(a, b, out, b_mn):
    g = _lib.SxGemmArgs()
    g.A, g.B, g.D = a.data_ptr(), b.data_ptr(), out.data_ptr() if out is not None else 0
    M, K = a.shape
    N = b.shape[1] if b_mn else b.shape[0]
    g.M, g.N, g.K, g.batch = M, N, K, 1
    g.lda, g.ldb, g.ldd = a.stride(0), b.stride(0), out.stride(0) if out is not None else N
    g.a_mn, g.b_mn = 0, int(b_mn)
    g.alpha, g.beta = 1.0, 0.0
    g.status = _lib.status_word(a.device).data_ptr()
    return g


class FusedTP:
    """Per-group workspace for the fused TP kernels: symmetric gather / staging buffers keyed by shape, flag arrays,
    epochs and reduce-scatter counter sites."""

    def __init__(self, sg, n_copy=None):
        self.sg = sg
        self.rank, self.world = sg.rank, sg.world
        # copy CTAs of the all-gather form: one remote chunk at a time is pulled by all of them; with more than two
        # ranks most of the operand is remote and the pull, not the GEMM, sets the pace
        self.n_copy = n_copy if n_copy is not None else (8 if sg.world <= 2 else 16)
        self._gather = {}
        self._stage = {}
        self._rs_sites = {}
        self._next_word = RS_COUNTER_WORD0
        self._ag_epoch = 0
        self._rs_epoch = 0
        self.cta_counter = torch.zeros(4, dtype=torch.int32, device=sg.device)

    def gather_buffer(self, rows_total, cols, dtype=torch.bfloat16, key=None):
        k = (key, rows_total, cols)
        if k not in self._gather:
            buf = self.sg.alloc(rows_total * cols, dtype)
            sub = 256 if (rows_total // self.world) % 256 == 0 else 128
            # sized for the finest sub-block (128 rows): ag_gemm may signal at a finer grain than `sub`
            flags = torch.zeros(self.world * max(1, (rows_total // self.world) // 128), dtype=torch.int32,
                                device=self.sg.device)
            self._gather[k] = (buf, flags, sub)
        return self._gather[k]

    def ag_gemm(self, x_shard, w, b_mn=False, key=None, gather_b=False):
        """(all-gather of row shards) x W^T in one kernel. ``x_shard`` [rows/world, K] is this rank's chunk of the
        gathered operand; returns (out, gathered) where ``gathered`` is the full operand (a view of the symmetric
        buffer, valid until the next call with the same key). With ``gather_b`` the roles swap: ``x_shard`` is this
        rank's row shard of the weight [N/world, K] and ``w`` is the local activation [M, K] (F2)."""
        rows_s, K = x_shard.shape
        rows = rows_s * self.world
        buf, flags, sub = self.gather_buffer(rows, K, x_shard.dtype, key)
        full = buf.tensor.view(rows, K)
        full[self.rank * rows_s: (self.rank + 1) * rows_s].copy_(x_shard)
        self._ag_epoch += 1
        if not gather_b and self.world > 2 and rows_s % 128 == 0:
            # many ranks, short chunks: 128-row sub-blocks give the copy CTAs (world - 1) * rows_s / 128 work items to
            # share and let a tile start as soon as its own 128 rows are in
            sub = 128
        if gather_b:
            act = w
            out = torch.empty(act.shape[0], rows, dtype=act.dtype, device=act.device)
            g = _gemm_args(act, full, out, False)
        else:
            N = w.shape[1] if b_mn else w.shape[0]
            out = torch.empty(rows, N, dtype=x_shard.dtype, device=x_shard.device)
            g = _gemm_args(full, w, out, b_mn)
        cm = SxGemmCommArgs()
        cm.peers = self.sg.peers(buf)
        cm.mode = 2 if gather_b else 1
        cm.flags = flags.data_ptr()
        cm.epoch = self._ag_epoch
        cm.n_copy = self.n_copy
        cm.chunk_rows, cm.sub_rows = rows_s, min(sub, rows_s)
        cm.sig_channel, cm.done_channel = AG_SIG, AG_DONE
        cm.cta_counter = self.cta_counter.data_ptr()
        _lib.call("sx_gemm_bf16_comm", C.byref(g), C.byref(cm), _lib.stream())
        return out, full

    def gemm_rs(self, x, w, b_mn=False, residual=None):
        """x [T, K_local] x W^T summed over ranks, rows scattered: returns this rank's [T/world, N] (+ residual)."""
        T, K = x.shape
        N = w.shape[1] if b_mn else w.shape[0]
        rows_s = T // self.world
        k = (T, N)
        if k not in self._stage:
            self._stage[k] = self.sg.alloc(self.world * rows_s * N, x.dtype)
        stage = self._stage[k]
        if k not in self._rs_sites:
            nblk = rows_s // 128
            self._rs_sites[k] = [self._next_word, 0]
            self._next_word += nblk
            assert self._next_word <= 48 * 16, "out of reduce-scatter counter words"
        site = self._rs_sites[k]
        bn = 256 if N > 128 else 128
        site[1] = (site[1] + 4 * ((N + bn - 1) // bn) * self.world) & 0xFFFFFFFF
        self._rs_epoch += 1
        out = torch.empty(rows_s, N, dtype=x.dtype, device=x.device)
        g = _gemm_args(x, w, None, b_mn)
        g.D = stage.tensor.data_ptr()
        cm = SxGemmCommArgs()
        cm.peers = self.sg.peers(stage)
        cm.mode = 3
        cm.epoch = self._rs_epoch
        cm.chunk_rows, cm.sub_rows = rows_s, 128
        cm.done_channel = RS_DONE
        cm.counter_word, cm.rs_expected = site[0], site[1]
        cm.rs_out, cm.rs_ldd = out.data_ptr(), out.stride(0)
        cm.rs_residual = residual.data_ptr() if residual is not None else None
        cm.cta_counter = self.cta_counter.data_ptr() + 4
        _lib.call("sx_gemm_bf16_comm", C.byref(g), C.byref(cm), _lib.stream())
        return out


# ----------------------------------------------------------------------------- library (baseline) collectives
def _all_gather_rows(x, group):
    w = dist.get_world_size(group)
    out = torch.empty(w * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


def _reduce_scatter_rows(x, group):
    w = dist.get_world_size(group)
    out = torch.empty(x.shape[0] // w, *x.shape[1:], dtype=x.dtype, device=x.device)
    if dist.get_backend(group) == "nccl":
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
    else:
        xf = x.float().contiguous()
        dist.all_reduce(xf, group=group)
        r = dist.get_rank(group)
        out.copy_(xf[r * out.shape[0]: (r + 1) * out.shape[0]])
    return out


class _ColumnParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_s, w, tp):
        if tp.fused is not None:
            y, full = tp.fused.ag_gemm(x_s, w, key="col")
            full = full.clone()
        else:
            full = _all_gather_rows(x_s, tp.group)
            y = gemm(full, w)
        ctx.save_for_backward(full, w)
        ctx.tp = tp
        return y

    @staticmethod
    def backward(ctx, dy):
        full, w = ctx.saved_tensors
        tp = ctx.tp
        dy = dy.contiguous()
        if tp.fused is not None:
            dx_s = tp.fused.gemm_rs(dy, w, b_mn=True)
        else:
            dx_s = _reduce_scatter_rows(gemm(dy, w, b_mn=True), tp.group)
        mg = getattr(w, "main_grad", None)
        if mg is not None:
            first = not getattr(w, "_main_grad_written", False)
            gemm(dy, full, a_mn=True, b_mn=True, out=mg, c=None if first else mg, beta=0.0 if first else 1.0)
            w._main_grad_written = True
            dw = None
        else:
            dw = gemm(dy, full, a_mn=True, b_mn=True, out_dtype=w.dtype)
        return dx_s, dw, None


class _RowParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, tp, residual):
        if tp.fused is not None:
            y_s = tp.fused.gemm_rs(x, w, residual=residual)
        else:
            y_s = _reduce_scatter_rows(gemm(x, w), tp.group)
            if residual is not None:
                y_s = y_s + residual
        ctx.save_for_backward(x, w)
        ctx.tp, ctx.has_res = tp, residual is not None
        return y_s

    @staticmethod
    def backward(ctx, dy_s):
        x, w = ctx.saved_tensors
        tp = ctx.tp
        dy_s = dy_s.contiguous()
        if tp.fused is not None:
            dx, dy_full = tp.fused.ag_gemm(dy_s, w, b_mn=True, key="row_bwd")
        else:
            dy_full = _all_gather_rows(dy_s, tp.group)
            dx = gemm(dy_full, w, b_mn=True)
        mg = getattr(w, "main_grad", None)
        if mg is not None:
            first = not getattr(w, "_main_grad_written", False)
            gemm(dy_full, x, a_mn=True, b_mn=True, out=mg, c=None if first else mg, beta=0.0 if first else 1.0)
            w._main_grad_written = True
            dw = None
        else:
            dw = gemm(dy_full, x, a_mn=True, b_mn=True, out_dtype=w.dtype)
        return dx, dw, None, (dy_s if ctx.has_res else None)


class TPContext:
    """Process group + (optionally) the fused workspace shared by all TP layers of a model."""

    def __init__(self, group=None, fused=None, sg=None):
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        use_fused = torch.cuda.is_available() and dist.get_backend(self.group) == "nccl" if fused is None else fused
        self.fused = None
        if use_fused and self.world > 1:
            from .symm import SymmGroup
            self.fused = FusedTP(sg or SymmGroup(self.group))


class ColumnParallelLinear(Module):
    """y[T, N/tp] = all_gather(x[T/tp, K]) W_local^T."""

    def __init__(self, in_features, out_features, tp: TPContext, dtype=None, device=None, init_std=0.02):
        super().__init__()
        assert out_features % tp.world == 0
        self.tp = tp
        self.weight = tnn.Parameter(torch.empty(out_features // tp.world, in_features, dtype=dtype, device=device))
        tnn.init.normal_(self.weight, std=init_std)
        self.weight.tensor_parallel = "column"

    def forward(self, x_s):
        shp = x_s.shape
        y = _ColumnParallelFn.apply(x_s.reshape(-1, shp[-1]), self.weight, self.tp)
        return y


class RowParallelLinear(Module):
    """y[T/tp, N] = reduce_scatter(x[T, K/tp] W_local^T) (+ residual)."""

    def __init__(self, in_features, out_features, tp: TPContext, dtype=None, device=None, init_std=0.02):
        super().__init__()
        assert in_features % tp.world == 0
        self.tp = tp
        self.weight = tnn.Parameter(torch.empty(out_features, in_features // tp.world, dtype=dtype, device=device))
        tnn.init.normal_(self.weight, std=init_std)
        self.weight.tensor_parallel = "row"

    def forward(self, x, residual=None):
        return _RowParallelFn.apply(x.reshape(-1, x.shape[-1]), self.weight, self.tp, residual)
