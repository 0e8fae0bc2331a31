"""HSS — hierarchical state space layer with a full state matrix, as the reference defines it
(algorithms/hss/core/discretize.c:98-134, scan.c:53-223, step.c:26, model.c:30-92; Python twin ``algo_hss.py``).

Parameters per layer (nine, like ``SNEPPX_hss_get_params``): x_proj weight and bias, LayerNorm weight and bias,
A [s, s], B [s, i], C [o, s], D [o, i], dt [s].  Discretisation scales ROW r of A and B by dt[r].

The reference scans token by token (O(L s^2) sequential).  Here the scan is GEMM-shaped so that it runs on the tensor
cores: U = X B_bar^T is one GEMM over all tokens, the recurrence h_t = A_bar h_{t-1} + u_t is solved by recursive
doubling  H <- H + shift_{2^k}(H) (A_bar^{2^k})^T  in ceil(log2 L) batched GEMMs, and Y = [H, X] [C, D]^T is one more.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as tnn

from ..nn.modules import LayerNorm, Linear, Module
from ..ops import ssm as ssm_ops


class HSSDiscretize:
    """Continuous (A, B, dt) -> discrete (A_bar, B_bar)."""

    @staticmethod
    def euler(A, B, dt):
        """A_bar = I + diag(dt) A, B_bar = diag(dt) B (discretize.c:98-134)."""
        s = A.shape[0]
        return torch.eye(s, dtype=A.dtype, device=A.device) + dt[:, None] * A, dt[:, None] * B

    @staticmethod
    def zoh(A, B, dt):
        """Zero-order hold: A_bar = exp(diag(dt) A), B_bar = (diag(dt) A)^-1 (A_bar - I) diag(dt) B."""
        s = A.shape[0]
        Ad = dt[:, None] * A
        A_bar = torch.matrix_exp(Ad)
        eye = torch.eye(s, dtype=A.dtype, device=A.device)
        B_bar = torch.linalg.solve(Ad, (A_bar - eye) @ (dt[:, None] * B))
        return A_bar, B_bar

    @staticmethod
    def bilinear(A, B, dt):
        """Tustin: A_bar = (I - Ad/2)^-1 (I + Ad/2), B_bar = (I - Ad/2)^-1 diag(dt) B."""
        s = A.shape[0]
        eye = torch.eye(s, dtype=A.dtype, device=A.device)
        Ad = dt[:, None] * A
        inv = torch.linalg.inv(eye - 0.5 * Ad)
        return inv @ (eye + 0.5 * Ad), inv @ (dt[:, None] * B)


class HSSScan:
    @staticmethod
    def sequential(A_bar, B_bar, C, D, x, h0=None):
        """Reference order of operations (scan.c:53-102). x [.., L, i] -> (y [.., L, o], h_last [.., s])."""
        lead, L = x.shape[:-2], x.shape[-2]
        h = x.new_zeros(*lead, A_bar.shape[0]) if h0 is None else h0
        ys = []
        for t in range(L):
            h = h @ A_bar.T + x[..., t, :] @ B_bar.T
            ys.append(h @ C.T + x[..., t, :] @ D.T)
        return torch.stack(ys, dim=-2), h

    @staticmethod
    def parallel_scan(A_bar, B_bar, C, D, x, h0=None, return_states=False):
        """Recursive doubling over the sequence; equal to ``sequential`` up to rounding (the reference's Blelloch
        scan over (A, b) pairs, scan.c:111-223, specialised to a constant A so that each level is one GEMM)."""
        L = x.shape[-2]
        H = x @ B_bar.T.to(x.dtype)                                     # u_t, [.., L, s]
        if h0 is not None:
            H = torch.cat([H[..., :1, :] + (h0 @ A_bar.T.to(x.dtype)).unsqueeze(-2), H[..., 1:, :]], dim=-2)
        P = A_bar.T.to(x.dtype)
        shift = 1
        while shift < L:
            moved = H[..., :-shift, :] @ P
            H = torch.cat([H[..., :shift, :], H[..., shift:, :] + moved], dim=-2)
            P = P @ P
            shift *= 2
        y = H @ C.T.to(x.dtype) + x @ D.T.to(x.dtype)
        return (y, H) if return_states else (y, H[..., -1, :])

    @staticmethod
    def selective_scan(x, dt, A, Bm, Cm, D=None, chunk=64):
        """Input-dependent (diagonal) scan: the chunked SSD path (``ops.ssm.ssd_scan``)."""
        return ssm_ops.ssd_scan(x, dt, A, Bm, Cm, D, chunk=chunk)


class HSSStep:
    @staticmethod
    def step(h, x, A_bar, B_bar, C, D):
        """One recurrent step (step.c:26): returns (y, h_next)."""
        h = h @ A_bar.T + x @ B_bar.T
        return h @ C.T + x @ D.T, h


@dataclass
class HSSConfig:
    """Defaults of ``SNEPPX_hss_config_default`` (algorithms/hss/core/layer.c:29-41)."""
    state_dim: int = 64
    input_dim: int = 512
    output_dim: int = 512
    num_layers: int = 2
    seq_len: int = 1024
    dt_min: float = 1e-3
    dt_max: float = 0.1
    discretization: str = "euler"
    scan: str = "parallel"


class DenseHSSLayer(Module):
    def __init__(self, cfg: HSSConfig = None, dtype=None, device=None, **kw):
        super().__init__()
        cfg = cfg or HSSConfig(**kw)
        self.cfg = cfg
        s, i, o = cfg.state_dim, cfg.input_dim, cfg.output_dim
        self.x_proj = Linear(i, i, bias=True, dtype=dtype, device=device)
        self.norm = LayerNorm(i, dtype=dtype, device=device)
        # Stable start: A = -(positive diagonal) + small coupling, so that I + dt A contracts for dt <= dt_max.
        A = -torch.diag(torch.empty(s).uniform_(0.5, 1.5)) + 0.01 * torch.randn(s, s)
        self.A = tnn.Parameter(A.to(device=device))
        self.B = tnn.Parameter((torch.randn(s, i) / math.sqrt(i)).to(device=device))
        self.C = tnn.Parameter((torch.randn(o, s) / math.sqrt(s)).to(device=device))
        self.D = tnn.Parameter((torch.randn(o, i) * 0.02).to(device=device))
        dt = torch.exp(torch.rand(s) * (math.log(cfg.dt_max) - math.log(cfg.dt_min)) + math.log(cfg.dt_min))
        self.dt = tnn.Parameter(dt.to(device=device))

    def discretize(self):
        return getattr(HSSDiscretize, self.cfg.discretization)(self.A.float(), self.B.float(), self.dt.float())

    def forward(self, x, h0=None, return_state=False):
        u = self.norm(self.x_proj(x))
        A_bar, B_bar = self.discretize()
        fn = HSSScan.parallel_scan if self.cfg.scan == "parallel" else HSSScan.sequential
        y, h = fn(A_bar.to(u.dtype), B_bar.to(u.dtype), self.C.to(u.dtype), self.D.to(u.dtype), u, h0)
        return (y, h) if return_state else y

    def step(self, x_t, h):
        """Single-token decode; x_t [.., i], h [.., s]."""
        u = self.norm(self.x_proj(x_t))
        A_bar, B_bar = self.discretize()
        return HSSStep.step(h, u, A_bar.to(u.dtype), B_bar.to(u.dtype), self.C.to(u.dtype), self.D.to(u.dtype))


class HSSModel(Module):
    """Stack of dense HSS layers (model.c:30-92); layer l>0 takes the previous layer's output width."""

    def __init__(self, cfg: HSSConfig = None, dtype=None, device=None, **kw):
        super().__init__()
        cfg = cfg or HSSConfig(**kw)
        self.cfg = cfg
        layers, i = [], cfg.input_dim
        for _ in range(cfg.num_layers):
            lc = HSSConfig(**{**cfg.__dict__, "input_dim": i})
            layers.append(DenseHSSLayer(lc, dtype=dtype, device=device))
            i = cfg.output_dim
        self.layers = tnn.ModuleList(layers)

    def forward(self, x):
        from ..utils.observability import bench_marker
        bench_marker("HSS forward start")
        for layer in self.layers:
            x = layer(x)
        bench_marker("HSS forward done")
        return x

    def num_params_per_layer(self):
        return len(list(self.layers[0].parameters()))
