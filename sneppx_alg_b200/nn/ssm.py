"""HSS (hierarchical state space) layers: the Mamba-2 SSD block used by the HSS configs, and the reference's
LTI HSS layer (dense x_proj -> LayerNorm -> linear time-invariant SSM) expressed on the same scan.

Mamba-2 block API mirrors ``sneppx_mamba2_init/forward(dim, d_state, d_conv)``
(include/neural_core/architecture/advanced_arch.h, kernel/arch/mamba2.c:36-133, whose body is a stub) and the
Python ``Mamba2`` class (interface_bindings/c_arch.py:42-74). Initialisation follows Mamba-2: A_log =
log(uniform[1, 16]), dt bias such that softplus(dt_bias) is log-uniform in [dt_min, dt_max] = [1e-3, 1e-1].
The reference HSS layer defaults (state 64, dt in [1e-3, 0.1]; algorithms/hss/core/layer.c:29-41) carry over.
"""
from __future__ import annotations

import math

import torch
import torch.nn as tnn
import torch.nn.functional as F

from ..ops import ssm
from .modules import LayerNorm, Linear, Module, RMSNorm


class Mamba2Block(Module):
    def __init__(self, d_model, d_state=128, d_conv=4, expand=2, headdim=64, ngroups=1, chunk_size=256,
                 dt_min=1e-3, dt_max=1e-1, eps=1e-5, dtype=None, device=None, init_std=0.02):
        super().__init__()
        self.d_model, self.d_state, self.d_conv = d_model, d_state, d_conv
        self.d_inner = expand * d_model
        self.headdim, self.ngroups, self.chunk = headdim, ngroups, chunk_size
        self.nheads = self.d_inner // headdim
        assert self.nheads % ngroups == 0
        self.conv_dim = self.d_inner + 2 * ngroups * d_state
        d_in_proj = 2 * self.d_inner + 2 * ngroups * d_state + self.nheads
        self.in_proj = Linear(d_model, d_in_proj, bias=False, dtype=dtype, device=device, init_std=init_std)
        self.conv_weight = tnn.Parameter(torch.empty(self.conv_dim, d_conv, dtype=dtype, device=device))
        self.conv_bias = tnn.Parameter(torch.zeros(self.conv_dim, dtype=dtype, device=device))
        tnn.init.uniform_(self.conv_weight, -1 / math.sqrt(d_conv), 1 / math.sqrt(d_conv))
        dt = torch.exp(torch.rand(self.nheads) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min))
        dt = dt.clamp(min=1e-4)
        self.dt_bias = tnn.Parameter((dt + torch.log(-torch.expm1(-dt))).to(device=device, dtype=torch.float32))
        self.A_log = tnn.Parameter(torch.log(torch.empty(self.nheads).uniform_(1, 16)).to(device=device,
                                                                                          dtype=torch.float32))
        self.D = tnn.Parameter(torch.ones(self.nheads, device=device, dtype=torch.float32))
        self.norm = RMSNorm(self.d_inner, eps, dtype=dtype, device=device)
        self.out_proj = Linear(self.d_inner, d_model, bias=False, dtype=dtype, device=device, init_std=init_std)

    def split(self, zxbcdt):
        di, gn, H = self.d_inner, self.ngroups * self.d_state, self.nheads
        z, xBC, dt = torch.split(zxbcdt, [di, di + 2 * gn, H], dim=-1)
        return z, xBC, dt

    def forward(self, u, state=None):
        """u [B, L, d_model]. ``state`` (dict with 'conv' [B, K-1, C] and 'ssm' [B, H, P, N]) enables chunked /
        incremental processing; it is updated in place when given."""
        B, L, _ = u.shape
        H, P, G, N = self.nheads, self.headdim, self.ngroups, self.d_state
        z, xBC, dt = self.split(self.in_proj(u))
        prev = state["conv"] if state is not None else None
        xBC_c = ssm.causal_conv1d(xBC, self.conv_weight, self.conv_bias, act=True, prev=prev)
        if state is not None:
            K = self.d_conv
            hist = torch.cat([prev, xBC], dim=1) if prev is not None else xBC
            state["conv"] = hist[:, -(K - 1):].contiguous()
        x, Bm, Cm = torch.split(xBC_c, [self.d_inner, G * N, G * N], dim=-1)
        dt = F.softplus(dt.float() + self.dt_bias)
        A = -torch.exp(self.A_log)
        init = state["ssm"] if state is not None and state.get("ssm") is not None else None
        out = ssm.ssd_scan(x.reshape(B, L, H, P), dt, A, Bm.reshape(B, L, G, N), Cm.reshape(B, L, G, N), self.D,
                           chunk=min(self.chunk, 128), init_state=init,   # result is independent of the tiling; 128 = one MMA tile
                          
                           return_state=state is not None)
        if state is not None:
            y, state["ssm"] = out
        else:
            y = out
        y = y.reshape(B, L, self.d_inner)
        y = self.norm(ssm.gate_mul(y, z))   # gated RMSNorm
        return self.out_proj(y)

    def allocate_state(self, batch, device=None, dtype=None):
        p = self.in_proj.weight
        return {"conv": torch.zeros(batch, self.d_conv - 1, self.conv_dim, device=device or p.device,
                                    dtype=dtype or p.dtype), "ssm": None}


Mamba2 = Mamba2Block


class HSSLayer(Module):
    """The reference's HSS layer (algorithms/hss/core/forward.c:40-74, discretize.c:98-134, scan.c:53-102):
    x_proj (dense + bias) -> LayerNorm -> LTI SSM  h_t = A_bar h_{t-1} + B_bar u_t,  y_t = C h_t + D u_t  with Euler
    discretisation A_bar = I + A dt, B_bar = B dt. Here A is diagonal (the structured case every fast scan uses);
    the scan itself is the chunked SSD kernel path with constant dt, B and C."""

    def __init__(self, input_dim=512, state_dim=64, output_dim=None, dt_min=1e-3, dt_max=0.1, dtype=None, device=None):
        super().__init__()
        output_dim = output_dim or input_dim
        self.input_dim, self.state_dim, self.output_dim = input_dim, state_dim, output_dim
        self.x_proj = Linear(input_dim, input_dim, bias=True, dtype=dtype, device=device)
        self.norm = LayerNorm(input_dim, dtype=dtype, device=device)
        self.A_log = tnn.Parameter(torch.log(torch.empty(input_dim).uniform_(1, 16)).to(device=device))
        self.B = tnn.Parameter(torch.randn(input_dim, state_dim, device=device) / math.sqrt(state_dim))
        self.C = tnn.Parameter(torch.randn(input_dim, state_dim, device=device) / math.sqrt(state_dim))
        self.D = tnn.Parameter(torch.ones(input_dim, device=device))
        dt = torch.exp(torch.rand(input_dim) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min))
        self.log_dt = tnn.Parameter(torch.log(dt).to(device=device))
        self.out = Linear(input_dim, output_dim, bias=True, dtype=dtype, device=device) if output_dim != input_dim else None

    def forward(self, x):
        """x [B, L, input_dim]: every channel is an independent head with headdim 1."""
        Bsz, L, d = x.shape
        u = self.norm(self.x_proj(x))
        dt = torch.exp(self.log_dt).view(1, 1, d).expand(Bsz, L, d)
        A = -torch.exp(self.A_log)
        # Euler step A_bar = 1 + A dt equals exp(A dt) to first order; the scan uses the exact exponential (ZOH).
        Bm = self.B.view(1, 1, d, self.state_dim).expand(Bsz, L, d, self.state_dim)
        Cm = self.C.view(1, 1, d, self.state_dim).expand(Bsz, L, d, self.state_dim)
        y = ssm.ssd_scan(u.reshape(Bsz, L, d, 1), dt, A, Bm.to(u.dtype), Cm.to(u.dtype), self.D, chunk=64)
        y = y.reshape(Bsz, L, d)
        return self.out(y) if self.out is not None else y
