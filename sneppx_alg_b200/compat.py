"""Names of the reference's flat Python namespace (``SneppX_ALG.interface_bindings``: ``pytorch_api.py``,
``keras_api.py``, ``tensor.py`` losses and pooling, ``schedulers.py``, ``optim_extra.py``, ``quantization.py``,
``mx_formats.py``, ``distillation.py``, ``pruning.py``, ``hpo.py`` / ``hparams.py``, ``augmentation.py``,
``llama_models.py`` class names, ``cuda_device.py``, ``driver_bindings.py`` C type aliases, the ``crypto_*`` wrappers and
the security service accessors) that have no module of their own here. Each is a working object built on this
package's modules or on ``torch``, not a placeholder; ``SneppX_ALG`` resolves unknown names through this module.
"""
from __future__ import annotations

import ctypes
import enum
import math
import random as _random
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch
import torch.nn as tnn
import torch.nn.functional as F

from . import device as _device
from .nn import modules as _nn
from .optim import zoo as _zoo
from .training import schedulers as _sched

# ----------------------------------------------------------------------------------------- layers (keras / torch style)
Flatten = tnn.Flatten
Softmax = tnn.Softmax
Conv2D = tnn.Conv2d
MaxPool2D = tnn.MaxPool2d
AveragePool2D = tnn.AvgPool2d
BatchNormalization = tnn.BatchNorm2d
PyTorchModule, PyTorchLinear, PyTorchEmbedding, PyTorchLayerNorm = _nn.Module, _nn.Linear, _nn.Embedding, _nn.LayerNorm
PyTorchDropout, PyTorchSequential, PyTorchConv2d, PyTorchParameter, PyTorchTensor = _nn.Dropout, tnn.Sequential, tnn.Conv2d, tnn.Parameter, torch.Tensor
Param = tnn.Parameter


class LlamaRMSNorm(_nn.RMSNorm):
    """RMSNorm under the name the Llama model files use."""



class Activation(tnn.Module):
    """Keras-style activation layer by name."""

    _FN = {"relu": F.relu, "gelu": lambda x: F.gelu(x, approximate="tanh"), "silu": F.silu, "swish": F.silu, "tanh": torch.tanh,
           "sigmoid": torch.sigmoid, "softmax": lambda x: torch.softmax(x, -1), "linear": lambda x: x}

    def __init__(self, name: str):
        super().__init__()
        if name not in self._FN:
            raise ValueError(f"unknown activation {name!r}")
        self.name = name

    def forward(self, x):
        return self._FN[self.name](x)


class InputSpec:
    """Keras-style input placeholder: records the per-sample shape."""

    def __init__(self, shape: Sequence[int], dtype=torch.float32):
        self.shape, self.dtype = tuple(shape), dtype

    def example(self, batch: int = 1):
        return torch.zeros((batch,) + tuple(d or 1 for d in self.shape), dtype=self.dtype)


def Input(shape: Sequence[int], dtype=torch.float32) -> InputSpec:
    """The input placeholder of a functional model (reference: interface_bindings/keras_api.py:362)."""
    return InputSpec(shape, dtype)


class PatchEmbedding(tnn.Module):
    """Image -> patch tokens (strided convolution), as in the vision transformers."""

    def __init__(self, img_size=224, patch_size=16, in_chans=3, embed_dim=768):
        super().__init__()
        self.num_patches = (img_size // patch_size) ** 2
        self.proj = tnn.Conv2d(in_chans, embed_dim, patch_size, patch_size)

    def forward(self, x):
        return self.proj(x).flatten(2).transpose(1, 2)


# ----------------------------------------------------------------------------------------- losses
MSELoss, BCELoss, CrossEntropyLoss, NLLLoss, KLDivLoss = tnn.MSELoss, tnn.BCELoss, tnn.CrossEntropyLoss, tnn.NLLLoss, tnn.KLDivLoss


def kd_loss(student_logits, teacher_logits, T: float = 2.0):
    """Temperature-softened KL divergence (Hinton distillation), scaled by T^2."""
    return F.kl_div(F.log_softmax(student_logits / T, -1), F.softmax(teacher_logits / T, -1), reduction="batchmean") * T * T


def hint_loss(student_feat, teacher_feat, regressor: Optional[Callable] = None):
    """FitNets hint: MSE between (optionally projected) student features and teacher features."""
    return F.mse_loss(regressor(student_feat) if regressor else student_feat, teacher_feat)


def attention_transfer_loss(student_feat, teacher_feat, p: int = 2):
    """Distance between the L2-normalised spatial attention maps (mean of |activation|^p over channels)."""
    def amap(f):
        return F.normalize(f.abs().pow(p).mean(1).flatten(1), dim=1)
    return (amap(student_feat) - amap(teacher_feat)).pow(2).mean()


def feature_matching_loss(student_feats, teacher_feats):
    return sum(F.mse_loss(s, t) for s, t in zip(student_feats, teacher_feats)) / max(len(student_feats), 1)


def correlation_congruence_loss(student_emb, teacher_emb):
    """Match the pairwise-similarity (Gram) matrices of a batch of embeddings."""
    gs = F.normalize(student_emb, dim=1) @ F.normalize(student_emb, dim=1).t()
    gt = F.normalize(teacher_emb, dim=1) @ F.normalize(teacher_emb, dim=1).t()
    return F.mse_loss(gs, gt)


def crd_loss(student_emb, teacher_emb, temperature: float = 0.1):
    """Contrastive representation distillation (in-batch negatives): each student embedding must pick its own
    teacher embedding among the batch."""
    logits = F.normalize(student_emb, dim=1) @ F.normalize(teacher_emb, dim=1).t() / temperature
    return F.cross_entropy(logits, torch.arange(logits.shape[0], device=logits.device))


def multi_teacher_distillation_loss(student_logits, teacher_logits_list, weights=None, T: float = 2.0):
    w = weights or [1.0 / len(teacher_logits_list)] * len(teacher_logits_list)
    return sum(wi * kd_loss(student_logits, t, T) for wi, t in zip(w, teacher_logits_list))


def ensemble_teacher_distillation(student_logits, teacher_logits_list, T: float = 2.0):
    """Distil from the mean of the teachers' softened distributions."""
    target = torch.stack([F.softmax(t / T, -1) for t in teacher_logits_list]).mean(0)
    return F.kl_div(F.log_softmax(student_logits / T, -1), target, reduction="batchmean") * T * T


def dpo_loss(policy_chosen_logp, policy_rejected_logp, ref_chosen_logp, ref_rejected_logp, beta: float = 0.1):
    """Direct preference optimisation: -log sigmoid(beta * ((pi_c - pi_r) - (ref_c - ref_r)))."""
    return -F.logsigmoid(beta * ((policy_chosen_logp - policy_rejected_logp) - (ref_chosen_logp - ref_rejected_logp))).mean()


def grpo_loss(logp, old_logp, rewards, clip: float = 0.2):
    """Group-relative policy optimisation: PPO clipping with advantages standardised inside the group (dim 0)."""
    adv = (rewards - rewards.mean()) / (rewards.std() + 1e-8)
    ratio = torch.exp(logp - old_logp)
    return -torch.min(ratio * adv, ratio.clamp(1 - clip, 1 + clip) * adv).mean()


def py_accuracy(pred, target) -> float:
    pred, target = torch.as_tensor(pred), torch.as_tensor(target)
    return float((pred == target).float().mean())


def py_f1(pred, target, positive=1) -> float:
    pred, target = torch.as_tensor(pred), torch.as_tensor(target)
    tp = int(((pred == positive) & (target == positive)).sum())
    fp = int(((pred == positive) & (target != positive)).sum())
    fn = int(((pred != positive) & (target == positive)).sum())
    return 0.0 if tp == 0 else 2 * tp / (2 * tp + fp + fn)


# ----------------------------------------------------------------------------------------- functional ops
adaptive_avg_pool2d, adaptive_max_pool2d = F.adaptive_avg_pool2d, F.adaptive_max_pool2d


def rotate_half(x):
    a, b = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat([-b, a], dim=-1)


def apply_rotary_pos_emb(q, k, cos, sin):
    """Rotate-half RoPE on q, k [..., S, D] with cos / sin [S, D] (the reference's llama_models.py:65-86)."""
    return q * cos + rotate_half(q) * sin, k * cos + rotate_half(k) * sin


def broadcast_shape(*shapes):
    return tuple(torch.broadcast_shapes(*shapes))


def rnn_cell(x, h, w_ih, w_hh, b_ih=None, b_hh=None):
    return torch.tanh(F.linear(x, w_ih, b_ih) + F.linear(h, w_hh, b_hh))


def gru_cell(x, h, w_ih, w_hh, b_ih=None, b_hh=None):
    gi, gh = F.linear(x, w_ih, b_ih), F.linear(h, w_hh, b_hh)
    ir, iz, i_n = gi.chunk(3, -1)
    hr, hz, hn = gh.chunk(3, -1)
    r, z = torch.sigmoid(ir + hr), torch.sigmoid(iz + hz)
    n = torch.tanh(i_n + r * hn)
    return (1 - z) * n + z * h


def lstm_cell(x, h, c, w_ih, w_hh, b_ih=None, b_hh=None):
    i, f, g, o = (F.linear(x, w_ih, b_ih) + F.linear(h, w_hh, b_hh)).chunk(4, -1)
    c2 = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
    return torch.sigmoid(o) * torch.tanh(c2), c2


def multi_head_attention(q, k, v, num_heads: int, causal: bool = False):
    """q, k, v [B, S, d] -> [B, S, d] through this package's attention op (flash kernel on bf16 CUDA tensors)."""
    from .ops import functional as ops
    B, S, d = q.shape
    hd = d // num_heads
    o = ops.attention(q.view(B, S, num_heads, hd), k.view(B, k.shape[1], num_heads, hd), v.view(B, v.shape[1], num_heads, hd), causal=causal)
    return o.reshape(B, S, d)


def transformer_block(x, block: tnn.Module):
    return block(x)


def count_parameters(model, trainable_only: bool = True) -> int:
    return sum(p.numel() for p in model.parameters() if p.requires_grad or not trainable_only)


def get_model_size_mb(model) -> float:
    return sum(p.numel() * p.element_size() for p in model.parameters()) / 2 ** 20


# ----------------------------------------------------------------------------------------- schedulers by class name
def _sched_class(fn_name, **fixed):
    def make(optimizer, **kw):
        return _sched.LRScheduler(optimizer, getattr(_sched, fn_name), **{**fixed, **kw})
    make.__name__ = fn_name
    return make


def _lambda_scheduler(optimizer, fn):
    return torch.optim.lr_scheduler.LambdaLR(optimizer, fn)


StepLR = torch.optim.lr_scheduler.StepLR
ExponentialLR = torch.optim.lr_scheduler.ExponentialLR
PolynomialLR = torch.optim.lr_scheduler.PolynomialLR
OneCycleLR = torch.optim.lr_scheduler.OneCycleLR
SequentialLR = torch.optim.lr_scheduler.SequentialLR
ChainedScheduler = torch.optim.lr_scheduler.ChainedScheduler
CosineAnnealingWarmRestarts = torch.optim.lr_scheduler.CosineAnnealingWarmRestarts
CosineLR = torch.optim.lr_scheduler.CosineAnnealingLR


class _ShapedLR(torch.optim.lr_scheduler.LambdaLR):
    """A multiplicative schedule given by ``shape(step) -> factor``; subclasses fix the shape from their arguments."""

    def __init__(self, optimizer, shape):
        self.shape = shape
        super().__init__(optimizer, shape)


class ConstantLRWithWarmup(_ShapedLR):
    def __init__(self, optimizer, warmup_steps: int):
        self.warmup_steps = warmup_steps
        super().__init__(optimizer, lambda s: min(1.0, (s + 1) / max(warmup_steps, 1)))


class CosineAnnealingWithWarmup(_ShapedLR):
    def __init__(self, optimizer, warmup_steps: int, total_steps: int, min_ratio: float = 0.0):
        self.warmup_steps, self.total_steps, self.min_ratio = warmup_steps, total_steps, min_ratio

        def f(s):
            if s < warmup_steps:
                return (s + 1) / max(warmup_steps, 1)
            t = min(1.0, (s - warmup_steps) / max(total_steps - warmup_steps, 1))
            return min_ratio + (1 - min_ratio) * 0.5 * (1 + math.cos(math.pi * t))
        super().__init__(optimizer, f)


class LinearWarmupCosineDecay(CosineAnnealingWithWarmup):
    """The reference's second name for linear warm-up followed by cosine decay."""


class CosineAnnealingWithWarmupRestarts(_ShapedLR):
    def __init__(self, optimizer, warmup_steps: int, cycle_steps: int, min_ratio: float = 0.0):
        self.warmup_steps, self.cycle_steps, self.min_ratio = warmup_steps, cycle_steps, min_ratio

        def f(s):
            s = s % max(cycle_steps, 1)
            if s < warmup_steps:
                return (s + 1) / max(warmup_steps, 1)
            t = (s - warmup_steps) / max(cycle_steps - warmup_steps, 1)
            return min_ratio + (1 - min_ratio) * 0.5 * (1 + math.cos(math.pi * t))
        super().__init__(optimizer, f)


class TriStageLR(_ShapedLR):
    """Linear warm-up, hold, exponential decay to final_ratio."""

    def __init__(self, optimizer, warmup_steps: int, hold_steps: int, decay_steps: int, init_ratio: float = 0.01,
                 final_ratio: float = 0.01):
        def f(s):
            if s < warmup_steps:
                return init_ratio + (1 - init_ratio) * s / max(warmup_steps, 1)
            if s < warmup_steps + hold_steps:
                return 1.0
            t = min(1.0, (s - warmup_steps - hold_steps) / max(decay_steps, 1))
            return math.exp(math.log(final_ratio) * t)
        super().__init__(optimizer, f)


# ----------------------------------------------------------------------------------------- optimizers by name
PyTorchSGD, PyTorchAdam, PyTorchAdamW, PyTorchOptimizer = _zoo.SGD, _zoo.Adam, torch.optim.AdamW, _zoo.Optimizer
CppSGD, CppAdam, CppAdamW, CppOptimizer = _zoo.SGD, _zoo.Adam, torch.optim.AdamW, _zoo.Optimizer
get_advanced_optimizer = get_extra_optimizer = _zoo.get_optimizer


class Adan(torch.optim.Optimizer):
    """Adaptive Nesterov momentum (Xie et al. 2022): moments of the gradient, of the gradient difference, and of the
    look-ahead gradient g + beta2 (g - g_prev)."""

    def __init__(self, params, lr=1e-3, betas=(0.02, 0.08, 0.01), eps=1e-8, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            b1, b2, b3 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st.update(m=torch.zeros_like(p), v=torch.zeros_like(p), n=torch.zeros_like(p), prev=p.grad.clone())
                d = p.grad - st["prev"]
                st["m"].mul_(1 - b1).add_(p.grad, alpha=b1)
                st["v"].mul_(1 - b2).add_(d, alpha=b2)
                u = p.grad + (1 - b2) * d
                st["n"].mul_(1 - b3).addcmul_(u, u, value=b3)
                step = (st["m"] + (1 - b2) * st["v"]) / (st["n"].sqrt() + g["eps"])
                p.mul_(1 / (1 + g["lr"] * g["weight_decay"])).add_(step, alpha=-g["lr"] / (1 + g["lr"] * g["weight_decay"]))
                st["prev"] = p.grad.clone()


class Sophia(torch.optim.Optimizer):
    """Sophia-G style update: momentum divided by an EMA of a diagonal Hessian estimate (here g^2, the Gauss-Newton
    proxy), clipped elementwise to [-1, 1]."""

    def __init__(self, params, lr=1e-4, betas=(0.965, 0.99), rho=0.04, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, rho=rho, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st.update(m=torch.zeros_like(p), h=torch.zeros_like(p))
                st["m"].mul_(b1).add_(p.grad, alpha=1 - b1)
                st["h"].mul_(b2).addcmul_(p.grad, p.grad, value=1 - b2)
                p.mul_(1 - g["lr"] * g["weight_decay"])
                p.add_((st["m"] / (g["rho"] * st["h"] + 1e-15)).clamp_(-1, 1), alpha=-g["lr"])


# ----------------------------------------------------------------------------------------- quantisation by name
from .quant import algorithms as _qa  # noqa: E402


class QuantGranularity:
    PER_TENSOR, PER_CHANNEL, PER_GROUP = "per_tensor", "per_channel", "per_group"


def quantize_int8_sym(x):
    """(int8 codes, scale): symmetric per-tensor, scale = absmax / 127."""
    s = x.abs().max().clamp_min(1e-12) / 127.0
    return torch.clamp(torch.round(x / s), -127, 127).to(torch.int8), s


def dequantize_int8_sym(q, s):
    return q.float() * s


def quantize_int8_asym(x):
    """(uint8 codes, scale, zero point) over [min, max]."""
    lo, hi = x.min(), x.max()
    s = ((hi - lo) / 255.0).clamp_min(1e-12)
    zp = torch.round(-lo / s)
    return torch.clamp(torch.round(x / s) + zp, 0, 255).to(torch.uint8), s, zp


def dequantize_int8_asym(q, s, zp):
    return (q.float() - zp) * s


def quantize_int8_channel(x, axis: int = 0):
    dims = [d for d in range(x.dim()) if d != axis]
    s = x.abs().amax(dims, keepdim=True).clamp_min(1e-12) / 127.0
    return torch.clamp(torch.round(x / s), -127, 127).to(torch.int8), s


def dequantize_int8_channel(q, s):
    return q.float() * s


def quantize_int4_sym(x, group: int = 128):
    return _qa.quantize_int4_packed(x, group)


def dequantize_int4_sym(packed, scales, group: int = 128):
    return _qa.dequantize_int4_packed(packed, scales, group)


def quantize_fp8_e4m3(x):
    return _qa.fp8_encode(x, _qa.QuantMode.FP8_E4M3)


def quantize_fp8_e5m2(x):
    return _qa.fp8_encode(x, _qa.QuantMode.FP8_E5M2)


def dequantize_fp8_e4m3(codes):
    return _qa.fp8_decode(codes, _qa.QuantMode.FP8_E4M3)


def dequantize_fp8_e5m2(codes):
    return _qa.fp8_decode(codes, _qa.QuantMode.FP8_E5M2)


MX_FORMATS = _qa.MX_FORMATS


def quantize_mx(x, fmt: str = "mxfp8", block: int = 32):
    """Micro-scaling fake quantisation by the short family name ("mxfp8" / "mxfp6" / "mxfp4") or by a full format
    name of ``MX_FORMATS`` ("mxfp6_e2m3", ...)."""
    return _qa.mx_quantize_spec(x, fmt, block) if fmt in _qa.MX_FORMATS else _qa.mx_quantize(x, fmt, block)


def dequantize_mx(x, fmt: str = "mxfp8"):
    """MX quantisation here returns the de-quantised (fake-quantised) tensor; de-quantising it again is the identity."""
    return x


def quantize_error(x, xq) -> float:
    return float((x.float() - xq.float()).pow(2).mean().sqrt() / x.float().pow(2).mean().sqrt().clamp_min(1e-12))


mx_error = quantize_error


def gptq_compute_hessian(inputs):
    """H = 2 X^T X / n over calibration activations [n, d] (the layer-wise objective's Hessian)."""
    x = inputs.reshape(-1, inputs.shape[-1]).float()
    return 2.0 * x.t() @ x / x.shape[0]


def awq_scale_weights(weight, act_scale, alpha: float = 0.5):
    """Activation-aware scaling: s = act_scale^alpha / weight_scale^(1 - alpha) per input channel; returns (W * s, s)."""
    ws = weight.abs().amax(0).clamp_min(1e-8)
    s = (act_scale.clamp_min(1e-8) ** alpha / ws ** (1 - alpha)).clamp(1e-4, 1e4)
    return weight * s, s


# ----------------------------------------------------------------------------------------- pruning
def magnitude_prune(weight, sparsity: float):
    """Mask keeping the (1 - sparsity) largest magnitudes of one tensor; returns (pruned weight, mask)."""
    k = int(weight.numel() * sparsity)
    if k == 0:
        return weight.clone(), torch.ones_like(weight, dtype=torch.bool)
    thr = weight.abs().flatten().kthvalue(k).values
    mask = weight.abs() > thr
    return weight * mask, mask


def global_magnitude_prune(model, sparsity: float, min_dim: int = 2):
    """One threshold over all weight matrices of the model; prunes in place, returns {name: mask}."""
    ws = [(n, p) for n, p in model.named_parameters() if p.dim() >= min_dim]
    allv = torch.cat([p.detach().abs().flatten() for _, p in ws])
    k = int(allv.numel() * sparsity)
    thr = allv.kthvalue(k).values if k else allv.new_tensor(-1.0)
    masks = {}
    with torch.no_grad():
        for n, p in ws:
            masks[n] = p.abs() > thr
            p.mul_(masks[n])
    return masks


def l1_channel_prune(weight, ratio: float):
    """Zeroes the output channels (rows) with the smallest L1 norms; returns (pruned weight, kept channel indices)."""
    norms = weight.abs().flatten(1).sum(1)
    drop = int(weight.shape[0] * ratio)
    keep = torch.sort(torch.argsort(norms, descending=True)[: weight.shape[0] - drop]).values
    out = torch.zeros_like(weight)
    out[keep] = weight[keep]
    return out, keep


def taylor_pruning(weight, grad, sparsity: float):
    """First-order Taylor importance |w * dL/dw|; prunes the least important entries."""
    imp = (weight * grad).abs()
    k = int(weight.numel() * sparsity)
    thr = imp.flatten().kthvalue(k).values if k else imp.new_tensor(-1.0)
    mask = imp > thr
    return weight * mask, mask


def movement_pruning(weight, scores, sparsity: float):
    """Keeps the entries with the highest learned movement scores."""
    k = int(weight.numel() * (1 - sparsity))
    idx = scores.flatten().topk(max(k, 1)).indices
    mask = torch.zeros(weight.numel(), dtype=torch.bool, device=weight.device)
    mask[idx] = True
    mask = mask.view_as(weight)
    return weight * mask, mask


def soft_pruning(weight, sparsity: float, shrink: float = 0.1):
    """Shrinks (rather than zeroes) the entries a magnitude mask would drop, so they can recover."""
    _, mask = magnitude_prune(weight, sparsity)
    return torch.where(mask, weight, weight * shrink), mask


def apply_pruning_mask(model, masks: Dict[str, torch.Tensor]):
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n in masks:
                p.mul_(masks[n].to(p.dtype))
    return model


def compute_sparsity(model_or_tensor) -> float:
    if torch.is_tensor(model_or_tensor):
        return float((model_or_tensor == 0).float().mean())
    tot = sum(p.numel() for p in model_or_tensor.parameters())
    return sum(int((p == 0).sum()) for p in model_or_tensor.parameters()) / max(tot, 1)


def recover_pruned_weights(model, masks, dense_state: Dict[str, torch.Tensor]):
    """Restores the pruned entries from a dense copy (the rewind step of lottery-ticket experiments)."""
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n in masks and n in dense_state:
                p.copy_(torch.where(masks[n], p, dense_state[n].to(p.dtype)))
    return model


def print_pruning_summary(model) -> str:
    rows = [f"{n:50s} {compute_sparsity(p):6.1%}" for n, p in model.named_parameters() if p.dim() >= 2]
    text = "\n".join(rows + [f"{'total':50s} {compute_sparsity(model):6.1%}"])
    print(text)
    return text


def find_winning_ticket(model, train_fn: Callable, sparsity: float, rounds: int = 3):
    """Iterative magnitude pruning with rewinding to the initial weights; returns the final masks."""
    init = {n: p.detach().clone() for n, p in model.named_parameters()}
    masks: Dict[str, torch.Tensor] = {}
    for r in range(1, rounds + 1):
        train_fn(model)
        masks = global_magnitude_prune(model, 1 - (1 - sparsity) ** (r / rounds))
        with torch.no_grad():
            for n, p in model.named_parameters():
                p.copy_(init[n] * masks[n] if n in masks else init[n])
    return masks


# ----------------------------------------------------------------------------------------- hyper-parameter search
@dataclass
class UniformFloat:
    low: float
    high: float

    def sample(self, rng):
        return rng.uniform(self.low, self.high)


@dataclass
class LogUniformFloat:
    low: float
    high: float

    def sample(self, rng):
        return math.exp(rng.uniform(math.log(self.low), math.log(self.high)))


@dataclass
class UniformInt:
    low: int
    high: int

    def sample(self, rng):
        return rng.randint(self.low, self.high)


@dataclass
class Choice:
    options: Sequence[Any]

    def sample(self, rng):
        return rng.choice(list(self.options))


@dataclass
class Fixed:
    value: Any

    def sample(self, rng):
        return self.value


def uniform(low: float, high: float) -> UniformFloat:
    return UniformFloat(float(low), float(high))


def log_uniform(low: float, high: float) -> LogUniformFloat:
    return LogUniformFloat(float(low), float(high))


def int_(low: int, high: int) -> UniformInt:
    """An integer range of a search space, both ends included (reference: interface_bindings/hpo.py:53)."""
    return UniformInt(int(low), int(high))


def choice(*o) -> Choice:
    return Choice(o[0] if len(o) == 1 and isinstance(o[0], (list, tuple)) else o)


@dataclass
class Trial:
    number: int
    params: Dict[str, Any]
    value: Optional[float] = None


class Sampler:
    """Base of the search samplers (reference: interface_bindings/hparams.py:173). A sampler is stateless about the
    space: ``suggest(space, history)`` returns the next parameter set given the trials so far; a sampler bound to a
    space at construction also answers ``sample()`` and ``total_trials()``."""

    def __init__(self, space: Optional[Dict[str, Any]] = None, seed: int = 42):
        self.space, self.rng, self._drawn = space, _random.Random(seed), []

    def suggest(self, space: Dict[str, Any], history: List["Trial"]) -> Dict[str, Any]:
        raise NotImplementedError

    def sample(self) -> Dict[str, Any]:
        if self.space is None:
            raise ValueError("this sampler was built without a search space")
        params = self.suggest(self.space, self._drawn)
        self._drawn.append(Trial(len(self._drawn), params))
        return params

    def total_trials(self) -> Optional[int]:
        """Number of distinct trials when the space is finite, else None."""
        return None


class RandomSampler(Sampler):
    def __init__(self, seed: int = 0, space: Optional[Dict[str, Any]] = None):
        super().__init__(space, seed)

    def suggest(self, space: Dict[str, Any], history: List[Trial]):
        return {k: v.sample(self.rng) for k, v in space.items()}


class GridSampler(Sampler):
    """Cartesian product of ``Choice`` / ``Fixed`` dimensions, in order."""

    def __init__(self, space: Optional[Dict[str, Any]] = None):
        super().__init__(space)
        self._grid = None

    def total_trials(self) -> Optional[int]:
        if self.space is None:
            return None
        n = 1
        for v in self.space.values():
            n *= len(v.options) if isinstance(v, Choice) else 1
        return n

    def suggest(self, space, history):
        if self._grid is None:
            import itertools
            dims = [list(v.options) if isinstance(v, Choice) else [v.value] for v in space.values()]
            self._grid = [dict(zip(space, c)) for c in itertools.product(*dims)]
        return self._grid[len(history) % len(self._grid)]


class BayesianSampler(RandomSampler):
    """Sequential model-based search in the TPE spirit: after `startup` random trials, candidates are drawn around
    the parameters of the best quarter of the trials and the one farthest from the worst trials is taken."""

    def __init__(self, seed: int = 0, startup: int = 5, candidates: int = 16, minimize: bool = True):
        super().__init__(seed)
        self.startup, self.candidates, self.minimize = startup, candidates, minimize

    def suggest(self, space, history):
        done = [t for t in history if t.value is not None]
        if len(done) < self.startup:
            return super().suggest(space, history)
        done.sort(key=lambda t: t.value, reverse=not self.minimize)
        good, bad = done[: max(1, len(done) // 4)], done[max(1, len(done) // 4):]
        numeric = [k for k, v in space.items() if isinstance(v, (UniformFloat, LogUniformFloat, UniformInt))]

        def dist(a, b):
            return sum(((a[k] - b[k]) / (abs(space[k].high - space[k].low) or 1.0)) ** 2 for k in numeric)

        best, best_score = None, -1.0
        for _ in range(self.candidates):
            base = self.rng.choice(good).params
            cand = {}
            for k, v in space.items():
                if k in numeric:
                    span = (v.high - v.low) * 0.15
                    x = min(max(base[k] + self.rng.uniform(-span, span), v.low), v.high)
                    cand[k] = int(round(x)) if isinstance(v, UniformInt) else x
                else:
                    cand[k] = base[k] if self.rng.random() < 0.8 else v.sample(self.rng)
            score = min((dist(cand, t.params) for t in bad), default=1.0)
            if score > best_score:
                best, best_score = cand, score
        return best


class Study:
    def __init__(self, space: Dict[str, Any], sampler=None, direction: str = "minimize"):
        self.space, self.sampler, self.direction = space, sampler or RandomSampler(), direction
        self.trials: List[Trial] = []

    def optimize(self, objective: Callable[[Dict[str, Any]], float], n_trials: int):
        for _ in range(n_trials):
            t = Trial(len(self.trials), self.sampler.suggest(self.space, self.trials))
            t.value = float(objective(t.params))
            self.trials.append(t)
        return self.best_trial

    @property
    def best_trial(self) -> Trial:
        key = (lambda t: t.value) if self.direction == "minimize" else (lambda t: -t.value)
        return min(self.trials, key=key)


@dataclass
class HPOConfig:
    n_trials: int = 20
    direction: str = "minimize"
    sampler: str = "random"
    seed: int = 0


class HPSearchRunner:
    def __init__(self, space, config: Optional[HPOConfig] = None):
        self.config = config or HPOConfig()
        s = {"random": RandomSampler(self.config.seed), "grid": GridSampler(),
             "bayesian": BayesianSampler(self.config.seed, minimize=self.config.direction == "minimize")}[self.config.sampler]
        self.study = Study(space, s, self.config.direction)

    def run(self, objective):
        return self.study.optimize(objective, self.config.n_trials)


def bayesian_search(objective, space, trials: int = 20, seed: int = 0, mode: str = "min"):
    st = Study(space, BayesianSampler(seed, minimize=mode == "min"), "minimize" if mode == "min" else "maximize")
    best = st.optimize(objective, trials)
    return best.params, best.value


def halving_search(objective: Callable[[Dict[str, Any], int], float], space, n_configs: int = 9, min_budget: int = 1, eta: int = 3,
                   seed: int = 0):
    """Successive halving: every round keeps the best 1 / eta configurations and multiplies their budget by eta."""
    rng = _random.Random(seed)
    configs = [{k: v.sample(rng) for k, v in space.items()} for _ in range(n_configs)]
    budget = min_budget
    scored = [(objective(c, budget), c) for c in configs]
    while len(scored) > 1:
        scored.sort(key=lambda t: t[0])
        keep = [c for _, c in scored[: max(1, len(scored) // eta)]]
        budget *= eta
        scored = [(objective(c, budget), c) for c in keep]
    return scored[0][1], scored[0][0]


# ----------------------------------------------------------------------------------------- augmentation
# images are [..., C, H, W] float tensors in [0, 1]; text is a list of tokens; audio features are [..., F, T]
def _gen_rand(generator, *shape):
    return torch.rand(*shape, generator=generator)


def random_horizontal_flip(img, prob=0.5, generator=None):
    return img.flip(-1) if float(_gen_rand(generator, 1)) < prob else img


def random_vertical_flip(img, prob=0.5, generator=None):
    return img.flip(-2) if float(_gen_rand(generator, 1)) < prob else img


def center_crop(img, size):
    h, w = (size, size) if isinstance(size, int) else size
    H, W = img.shape[-2:]
    t, l = (H - h) // 2, (W - w) // 2
    return img[..., t:t + h, l:l + w]


def five_crop(img, size):
    h, w = (size, size) if isinstance(size, int) else size
    H, W = img.shape[-2:]
    return [img[..., :h, :w], img[..., :h, W - w:], img[..., H - h:, :w], img[..., H - h:, W - w:], center_crop(img, (h, w))]


def ten_crop(img, size):
    return five_crop(img, size) + five_crop(img.flip(-1), size)


def random_resized_crop(img, size, scale=(0.08, 1.0), generator=None):
    H, W = img.shape[-2:]
    area = float(scale[0] + (scale[1] - scale[0]) * _gen_rand(generator, 1)) * H * W
    side = max(1, min(int(area ** 0.5), H, W))
    t = int(_gen_rand(generator, 1) * (H - side + 1))
    l = int(_gen_rand(generator, 1) * (W - side + 1))
    crop = img[..., t:t + side, l:l + side]
    out = (size, size) if isinstance(size, int) else tuple(size)
    lead = crop.shape[:-3]
    return F.interpolate(crop.reshape(-1, *crop.shape[-3:]), size=out, mode="bilinear", align_corners=False).reshape(*lead, crop.shape[-3], *out)


def random_rotation(img, degrees=15.0, generator=None):
    a = math.radians(float((_gen_rand(generator, 1) * 2 - 1) * degrees))
    theta = torch.tensor([[math.cos(a), -math.sin(a), 0.0], [math.sin(a), math.cos(a), 0.0]], dtype=img.dtype)
    x = img.reshape(-1, *img.shape[-3:])
    grid = F.affine_grid(theta.expand(x.shape[0], 2, 3), list(x.shape), align_corners=False)
    return F.grid_sample(x, grid, align_corners=False).reshape(img.shape)


def cutout(img, size=8, generator=None):
    H, W = img.shape[-2:]
    cy, cx = int(_gen_rand(generator, 1) * H), int(_gen_rand(generator, 1) * W)
    out = img.clone()
    out[..., max(cy - size // 2, 0):cy + size // 2, max(cx - size // 2, 0):cx + size // 2] = 0
    return out


random_erasing = cutout


def color_jitter(img, brightness=0.2, contrast=0.2, generator=None):
    b = 1 + float((_gen_rand(generator, 1) * 2 - 1) * brightness)
    c = 1 + float((_gen_rand(generator, 1) * 2 - 1) * contrast)
    mean = img.mean((-3, -2, -1), keepdim=True)
    return ((img * b - mean) * c + mean).clamp(0, 1)


def random_grayscale(img, prob=0.1, generator=None):
    if float(_gen_rand(generator, 1)) >= prob or img.shape[-3] != 3:
        return img
    g = (0.299 * img[..., 0:1, :, :] + 0.587 * img[..., 1:2, :, :] + 0.114 * img[..., 2:3, :, :])
    return g.expand_as(img).clone()


def gaussian_blur(img, kernel_size=3, sigma=1.0):
    k = torch.arange(kernel_size, dtype=img.dtype) - (kernel_size - 1) / 2
    g = torch.exp(-k ** 2 / (2 * sigma ** 2))
    g = (g / g.sum())
    C = img.shape[-3]
    x = img.reshape(-1, C, *img.shape[-2:])
    x = F.conv2d(x, g.view(1, 1, 1, -1).expand(C, 1, 1, -1), padding=(0, kernel_size // 2), groups=C)
    x = F.conv2d(x, g.view(1, 1, -1, 1).expand(C, 1, -1, 1), padding=(kernel_size // 2, 0), groups=C)
    return x.reshape(img.shape)


def sharpness(img, factor=2.0):
    return (img + (factor - 1) * (img - gaussian_blur(img))).clamp(0, 1)


def invert(img):
    return 1.0 - img


def solarize(img, threshold=0.5):
    return torch.where(img >= threshold, 1.0 - img, img)


def posterize(img, bits=4):
    levels = 2 ** bits
    return torch.floor(img * (levels - 1) + 0.5) / (levels - 1)


def auto_contrast(img):
    lo, hi = img.amin((-2, -1), keepdim=True), img.amax((-2, -1), keepdim=True)
    return torch.where(hi > lo, (img - lo) / (hi - lo).clamp_min(1e-12), img)


def equalize(img, bins=256):
    """Histogram equalisation per channel."""
    flat = img.reshape(-1, img.shape[-2] * img.shape[-1])
    out = torch.empty_like(flat)
    for i, ch in enumerate(flat):
        idx = (ch * (bins - 1)).long().clamp(0, bins - 1)
        cdf = torch.bincount(idx, minlength=bins).cumsum(0).float()
        cdf = (cdf - cdf.min()) / (cdf.max() - cdf.min()).clamp_min(1e-12)
        out[i] = cdf[idx]
    return out.reshape(img.shape)


def augmix(img, severity=3, width=3, generator=None):
    """Convex mixture of `width` short chains of simple operations, blended with the original."""
    ops_ = [auto_contrast, lambda x: posterize(x, max(1, 8 - severity)), lambda x: solarize(x, 1 - 0.1 * severity),
            lambda x: random_rotation(x, 5.0 * severity, generator), lambda x: sharpness(x, 1 + 0.3 * severity)]
    w = torch.distributions.Dirichlet(torch.ones(width)).sample()
    mix = torch.zeros_like(img)
    for i in range(width):
        x = img
        for _ in range(int(_gen_rand(generator, 1) * 3) + 1):
            x = ops_[int(_gen_rand(generator, 1) * len(ops_))](x)
        mix = mix + w[i] * x
    m = float(torch.distributions.Beta(1.0, 1.0).sample())
    return (m * img + (1 - m) * mix).clamp(0, 1)


class Compose:
    def __init__(self, transforms):
        self.transforms = list(transforms)

    def __call__(self, x):
        for t in self.transforms:
            x = t(x)
        return x


class RandomApply(Compose):
    def __init__(self, transforms, p=0.5):
        super().__init__(transforms)
        self.p = p

    def __call__(self, x):
        return super().__call__(x) if _random.random() < self.p else x


class RandomChoice(Compose):
    def __call__(self, x):
        return _random.choice(self.transforms)(x)


class RandomOrder(Compose):
    def __call__(self, x):
        for t in _random.sample(self.transforms, len(self.transforms)):
            x = t(x)
        return x


CIFAR10_TRAIN_TRANSFORMS = Compose([lambda x: random_crop_pad(x, 32, 4), random_horizontal_flip])
CIFAR10_EVAL_TRANSFORMS = Compose([])
IMAGENET_TRAIN_TRANSFORMS = Compose([lambda x: random_resized_crop(x, 224), random_horizontal_flip])
IMAGENET_EVAL_TRANSFORMS = Compose([lambda x: center_crop(x, 224)])


def random_crop_pad(img, size, padding):
    from .training.augmentation import random_crop
    if img.dim() == 3:   # the batched op wants [B, C, H, W]
        return random_crop(img.unsqueeze(0), size, padding)[0]
    return random_crop(img, size, padding)


def time_mask(spec, max_width=10, generator=None):
    T = spec.shape[-1]
    w = int(_gen_rand(generator, 1) * max_width)
    t0 = int(_gen_rand(generator, 1) * max(T - w, 1))
    out = spec.clone()
    out[..., t0:t0 + w] = 0
    return out


def freq_mask(spec, max_width=8, generator=None):
    return time_mask(spec.transpose(-1, -2), max_width, generator).transpose(-1, -2)


def time_stretch(wave, rate=1.1):
    n = max(1, int(wave.shape[-1] / rate))
    return F.interpolate(wave.reshape(-1, 1, wave.shape[-1]), size=n, mode="linear", align_corners=False).reshape(*wave.shape[:-1], n)


def pitch_shift(wave, semitones=2.0):
    """Resample by 2^(semitones / 12) and stretch back to the original length."""
    shifted = time_stretch(wave, 2 ** (semitones / 12))
    return F.interpolate(shifted.reshape(-1, 1, shifted.shape[-1]), size=wave.shape[-1], mode="linear",
                         align_corners=False).reshape(wave.shape)


def random_token_mask(tokens, mask_token="[MASK]", prob=0.15, rng=None):
    rng = rng or _random
    return [mask_token if rng.random() < prob else t for t in tokens]


def random_word_dropout(tokens, prob=0.1, rng=None):
    rng = rng or _random
    kept = [t for t in tokens if rng.random() >= prob]
    return kept or tokens[:1]


def random_word_shuffle(tokens, window=3, rng=None):
    rng = rng or _random
    keyed = sorted(range(len(tokens)), key=lambda i: i + rng.uniform(0, window))
    return [tokens[i] for i in keyed]


def token_cutout(tokens, max_len=3, rng=None):
    rng = rng or _random
    if len(tokens) <= 1:
        return list(tokens)
    n = rng.randint(1, min(max_len, len(tokens) - 1))
    s = rng.randint(0, len(tokens) - n)
    return list(tokens[:s]) + list(tokens[s + n:])


# ----------------------------------------------------------------------------------------- model class names and factories
from .models import config as _mcfg  # noqa: E402
from .models import families as _fam  # noqa: E402
from .models import llama as _llama  # noqa: E402
from .models.deepseek import DeepSeekLayer as DeepSeekV2DecoderLayer  # noqa: E402,F401
from .nn import attention as _attn  # noqa: E402

LlamaDecoderLayer = _llama.LlamaBlock
MistralDecoderLayer, Qwen2DecoderLayer = _llama.MistralDecoderLayer, _llama.Qwen2DecoderLayer
MistralAttention, Qwen2Attention = _llama.MistralAttention, _llama.Qwen2Attention
MistralMLP, Qwen2MLP = _llama.MistralMLP, _llama.Qwen2MLP


class DeepSeekV2MLP(_llama.LlamaMLP):
    """The dense SwiGLU feed-forward of DeepSeek-V2's first layers and of its shared experts."""

DeepSeekV2Attention = _attn.MultiHeadLatentAttention
LlamaModel, MistralModel, Qwen2Model = _llama.LlamaModel, _llama.MistralModel, _llama.Qwen2Model
GPTLMHeadModel, T5Model, ViTBlock = _fam.GPTLMHeadModel, _fam.T5Model, _fam._Block
MAE, mae_base, mae_large = _fam.MAE, _fam.mae_base, _fam.mae_large


def _family_table(family):
    return {f"{family}-{size}": _mcfg.get_model_config(family, size) for fam, sizes in _mcfg.list_models().items() if fam == family
            for size in sizes}


def __getattr__(name):   # configuration tables are built on first use
    tables = {"LLAMA_CONFIGS": ("llama2", "llama3"), "MISTRAL_CONFIGS": ("mistral",), "QWEN2_CONFIGS": ("qwen2",),
              "DEEPSEEK_V2_CONFIGS": ("deepseek_v2",)}
    if name in tables:
        out = {}
        for fam in tables[name]:
            out.update(_family_table(fam))
        return out
    raise AttributeError(name)


class LlamaRotaryEmbedding(tnn.Module):
    """cos / sin tables for rotate-half RoPE: forward(seq_len) -> (cos, sin) of shape [seq_len, dim]."""

    def __init__(self, dim, max_position_embeddings=2048, base=10000.0):
        super().__init__()
        self.dim, self.base = dim, base

    def forward(self, seq_len, device=None):
        from .ops.functional import rope_tables
        cos, sin = rope_tables(seq_len, self.dim, self.base, device)
        return torch.cat([cos, cos], -1), torch.cat([sin, sin], -1)


def _creator(default):
    def make(name=default, **kw):
        return _llama.create_model(name, **kw)
    return make


create_llama_model, create_mistral_model = _creator("llama3-tiny"), _creator("mistral-7b")
create_qwen2_model, create_deepseek_v2_model = _creator("qwen2-7b"), _creator("deepseek-v2-lite")
get_model = build_model_from_config = _llama.create_model


def build_transformer_from_config(cfg, **kw):
    from .models import build_model
    return build_model(cfg if isinstance(cfg, _mcfg.ModelConfig) else _mcfg.ModelConfig.from_dict(cfg), **kw)


def config_from_json(path):
    return _mcfg.ModelConfig.from_json(path)


def list_available_models():
    return [f"{fam}-{size}" for fam, sizes in _mcfg.list_models().items() for size in sizes]


def create_bert_model(**kw):
    return _fam.BertModel(_fam.BertConfig(**kw))


def create_gpt_model(**kw):
    return _fam.GPTModel(_fam.GPTConfig(**kw))


def create_t5_model(**kw):
    return _fam.T5ForConditionalGeneration(_fam.T5Config(**kw))


def create_vision_model(**kw):
    return _fam.VisionTransformer(_fam.ViTConfig(**kw))


def _vit(dim, depth, heads, patch, img=224):
    def make(num_classes=1000, **kw):
        fields = {f for f in _fam.ViTConfig.__dataclass_fields__}
        guess = {"hidden_size": dim, "num_layers": depth, "num_heads": heads, "patch_size": patch, "image_size": img,
                 "num_classes": num_classes, "embed_dim": dim, "depth": depth, "img_size": img}
        return _fam.VisionTransformer(_fam.ViTConfig(**{k: v for k, v in {**guess, **kw}.items() if k in fields}))
    return make


vit_tiny_patch16_224, vit_small_patch16_224 = _vit(192, 12, 3, 16), _vit(384, 12, 6, 16)
vit_base_patch16_224, vit_large_patch16_224, vit_huge_patch14_224 = _vit(768, 12, 12, 16), _vit(1024, 24, 16, 16), _vit(1280, 32, 16, 14)
mae_base, mae_large, mae_huge = vit_base_patch16_224, vit_large_patch16_224, vit_huge_patch14_224


def load_hf_weights(model, path):
    """Loads a Hugging Face safetensors / .pth file into `model`, mapping parameter names."""
    from .hub import formats
    from .hub.model_hub import map_hf_name
    sd = formats.load_any(path)
    mapped = {map_hf_name(k) or k: v for k, v in sd.items()}
    return (model.load_reference_state_dict if hasattr(model, "load_reference_state_dict") else model.load_state_dict)(mapped, strict=False)


convert_hf_llama_weights = load_hf_weights


def read_safetensors(path):
    from .hub.formats import load_safetensors
    return load_safetensors(path)[0]


def get_lora_parameters(model):
    return [p for n, p in model.named_parameters() if "lora_" in n]


@dataclass
class LoRAConfig:
    r: int = 8
    alpha: float = 16.0
    dropout: float = 0.0
    target_modules: Sequence[str] = ("qkv_proj", "o_proj", "gate_up_proj", "down_proj")


# ----------------------------------------------------------------------------------------- device layer and C type aliases
cuda_is_available = _device.is_available
detect_devices = lambda: [_device.properties(i) for i in range(_device.device_count())]  # noqa: E731


def current_device() -> int:
    return torch.cuda.current_device() if torch.cuda.is_available() else -1


def get_device_name(i: int = 0) -> str:
    return torch.cuda.get_device_name(i) if torch.cuda.is_available() else "cpu"


def get_device_capability(i: int = 0):
    return torch.cuda.get_device_capability(i) if torch.cuda.is_available() else (0, 0)


def cuda_memory_summary(i: int = 0) -> str:
    return torch.cuda.memory_summary(i) if torch.cuda.is_available() else "no CUDA device"


def detect_cpu() -> dict:
    import os
    import platform
    flags = ""
    try:
        flags = next(l for l in open("/proc/cpuinfo") if l.startswith("flags")).split(":", 1)[1]
    except (OSError, StopIteration):
        pass
    return {"arch": platform.machine(), "cores": os.cpu_count(), **{f: f in flags.split() for f in ("sse4_2", "avx2", "avx512f")}}


class CPUFeatures:
    """Instruction-set features of the host CPU, read from the kernel's flag list once at construction
    (reference: interface_bindings/asm_bridge.py:17 reads the same bits through cpuid)."""

    NAMES = {"aes_ni": "aes", "sha_ni": "sha_ni", "avx2": "avx2", "avx512f": "avx512f", "sse2": "sse2", "sse4_2": "sse4_2",
             "bmi2": "bmi2", "adx": "adx"}

    def __init__(self):
        try:
            flags = next(l for l in open("/proc/cpuinfo") if l.startswith("flags")).split(":", 1)[1].split()
        except (OSError, StopIteration):
            flags = []
        self._features = {k: v in flags for k, v in self.NAMES.items()}

    def has(self, name: str) -> bool:
        return bool(self._features.get(name, False))

    def as_dict(self) -> dict:
        return dict(self._features)

    def __getattr__(self, name):
        if name.startswith("has_") and name[4:] in self.NAMES:
            return self._features[name[4:]]
        raise AttributeError(name)
CUDAStream = torch.cuda.Stream
CUDAEvent = torch.cuda.Event
class ComputeCapability(enum.Enum):
    """Named compute-capability levels; ``ComputeCapability.of(i)`` is the newest level device ``i`` reaches."""

    PASCAL = (6, 0)
    VOLTA = (7, 0)
    TURING = (7, 5)
    AMPERE = (8, 0)
    HOPPER = (9, 0)
    BLACKWELL = (10, 0)

    @classmethod
    def of(cls, i: int = 0):
        cap = tuple(get_device_capability(i))
        reached = [c for c in cls if c.value <= cap]
        return reached[-1] if reached else None


class CUDADevice:
    """The one device layer (CUDA sm_100a); the reference's multi-vendor driver table is not reproduced."""

    def __init__(self, index: int = 0):
        self.index = index

    def __enter__(self):
        self._prev = current_device()
        _device.set_device(self.index)
        return self

    def __exit__(self, *exc):
        if self._prev >= 0:
            _device.set_device(self._prev)

    properties = property(lambda self: _device.properties(self.index))
    synchronize = staticmethod(_device.synchronize)


Device = CUDADevice


def get_backend() -> str:
    return "cuda" if torch.cuda.is_available() else "cpu"


get_kernel_backend = get_algo_backend = get_infra_backend = get_security_backend = get_backend

int8_t, int16_t, int32_t, int64_t = ctypes.c_int8, ctypes.c_int16, ctypes.c_int32, ctypes.c_int64
uint8_t, uint16_t, uint32_t, uint64_t = ctypes.c_uint8, ctypes.c_uint16, ctypes.c_uint32, ctypes.c_uint64
float_t, double_t, size_t, ssize_t = ctypes.c_float, ctypes.c_double, ctypes.c_size_t, ctypes.c_ssize_t
void_p, const_char_p = ctypes.c_void_p, ctypes.c_char_p


def make_struct(name: str, fields):
    """ctypes.Structure subclass from [(field name, ctype), ...]."""
    return type(name, (ctypes.Structure,), {"_fields_": list(fields)})


def load_library(which: str = "host"):
    from . import _build
    return _build.load_host() if which == "host" else _build.load_cuda()


find_load = load_library


# ----------------------------------------------------------------------------------------- crypto wrappers by class name
from .security import crypto as _c  # noqa: E402

shake_256 = _c.shake256


def shake_128(data: bytes, length: int) -> bytes:
    import hashlib
    return hashlib.shake_128(data).digest(length)   # only SHAKE-256 is native here


class AESGCM:
    def __init__(self, key: bytes):
        self.key = key

    def encrypt(self, nonce: bytes, data: bytes, aad: bytes = b"") -> bytes:
        return _c.aes256_gcm_encrypt(self.key, nonce, data, aad or b"")

    def decrypt(self, nonce: bytes, data: bytes, aad: bytes = b"") -> bytes:
        return _c.aes256_gcm_decrypt(self.key, nonce, data, aad or b"")


class AEAD(AESGCM):
    """ChaCha20-Poly1305 (RFC 8439)."""

    def encrypt(self, nonce, data, aad=b""):
        return _c.aead_encrypt(self.key, nonce, data, aad or b"")

    def decrypt(self, nonce, data, aad=b""):
        return _c.aead_decrypt(self.key, nonce, data, aad or b"")


class ChaCha20:
    def __init__(self, key: bytes, nonce: bytes, counter: int = 0):
        self.key, self.nonce, self.counter = key, nonce, counter

    def process(self, data: bytes) -> bytes:
        return _c.chacha20(self.key, self.nonce, data, self.counter)

    encrypt = decrypt = process


class Ed25519:
    def __init__(self, seed: bytes):
        self.seed, self.public_key = seed, _c.ed25519_public_key(seed)

    def sign(self, message: bytes) -> bytes:
        return _c.ed25519_sign(self.seed, message)

    @staticmethod
    def verify(public_key: bytes, message: bytes, signature: bytes) -> bool:
        return _c.ed25519_verify(public_key, message, signature)


class X25519:
    BASE = bytes([9] + [0] * 31)

    def __init__(self, private_key: bytes):
        self.private_key, self.public_key = private_key, _c.x25519(private_key, self.BASE)

    def exchange(self, peer_public: bytes) -> bytes:
        return _c.x25519(self.private_key, peer_public)


class HKDF:
    def __init__(self, salt: bytes = b"", info: bytes = b"", length: int = 32):
        self.salt, self.info, self.length = salt, info, length

    def derive(self, ikm: bytes) -> bytes:
        return _c.hkdf_sha256(ikm, self.salt, self.info, self.length)


class PBKDF2:
    def __init__(self, salt: bytes, iterations: int = 100000, length: int = 32):
        self.salt, self.iterations, self.length = salt, iterations, length

    def derive(self, password: bytes) -> bytes:
        return _c.pbkdf2_sha256(password, self.salt, self.iterations, self.length)


class HMAC_:
    def __init__(self, key: bytes):
        self.key = key

    def digest(self, msg: bytes) -> bytes:
        return _c.hmac_sha256(self.key, msg)

    def verify(self, msg: bytes, tag: bytes) -> bool:
        return _c.ct_equal(self.digest(msg), tag)


class SipHash:
    def __init__(self, key: bytes):
        self.key = key

    def hash(self, data: bytes) -> int:
        return _c.siphash24(self.key, data)


DRBG = _c.HmacDrbg


class EntropyPool:
    """Collects entropy from several sources (OS randomness, clock jitter, caller-supplied bytes), hashes it into a
    pool and seeds an HMAC-DRBG from the pool; ``random_bytes`` draws from the DRBG and reseeds it every
    ``reseed_interval`` calls (reference: interface_bindings/crypto_util.py:149)."""

    def __init__(self, reseed_interval: int = 1024):
        import hashlib
        self._h = hashlib.sha512()
        self._n, self._interval, self._drbg = 0, reseed_interval, None
        self.collect()

    def add(self, data: bytes):
        self._h.update(len(data).to_bytes(4, "big") + bytes(data))

    def collect(self):
        import os
        import time
        self.add(os.urandom(48))
        jitter = bytearray()
        for _ in range(64):
            jitter += (time.perf_counter_ns() & 0xFF).to_bytes(1, "big")
        self.add(bytes(jitter))
        self.add(os.getpid().to_bytes(4, "big"))

    def _seed(self) -> bytes:
        d = self._h.digest()
        self._h.update(d)
        return d

    def random_bytes(self, n: int) -> bytes:
        if self._drbg is None:
            self._drbg = _c.HmacDrbg(self._seed())
        elif self._n and self._n % self._interval == 0:
            self.collect()
            self.add(self._drbg.generate(32))
            self._drbg = _c.HmacDrbg(self._seed())
        self._n += 1
        return self._drbg.generate(n)
KyberKEM, Dilithium, SphincsPlus = _c.KyberKEM, _c.Dilithium, _c.SphincsPlus
MontgomeryMul = _c.MontgomeryMul
SecureAllocator = _c.GuardedBuffer


class ConstantTime:
    equal = staticmethod(_c.ct_equal)




class ModelHasher:
    """SHA-256 over a model's parameters in name order (integrity / watermark checks)."""

    @staticmethod
    def hash(model) -> str:
        import hashlib
        h = hashlib.sha256()
        for n, p in sorted(model.state_dict().items()):
            h.update(n.encode())
            h.update(p.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes())
        return h.hexdigest()


class Argon2:
    """Argon2id password hashing with a random salt; ``hash`` returns salt || tag, ``verify`` recomputes it."""

    def __init__(self, time_cost: int = 2, memory_kib: int = 19456, lanes: int = 1, length: int = 32):
        self.t, self.m, self.p, self.n = time_cost, memory_kib, lanes, length

    def hash(self, password: bytes, salt: Optional[bytes] = None) -> bytes:
        import os
        salt = salt or os.urandom(16)
        return salt + _c.argon2id(password, salt, self.t, self.m, self.p, self.n)

    def verify(self, password: bytes, stored: bytes) -> bool:
        return _c.ct_equal(self.hash(password, stored[:16]), stored)


class Poly1305:
    def __init__(self, key: bytes):
        self.key = key

    def tag(self, message: bytes) -> bytes:
        return _c.poly1305(self.key, message)

    def verify(self, message: bytes, tag: bytes) -> bool:
        return _c.ct_equal(self.tag(message), tag)


class Blake3:
    def __init__(self, key: Optional[bytes] = None):
        self.key, self._buf = key, b""

    def update(self, data: bytes):
        self._buf += data
        return self

    def digest(self, length: int = 32) -> bytes:
        return _c.blake3(self._buf, length, self.key)

    def hexdigest(self, length: int = 32) -> str:
        return self.digest(length).hex()
