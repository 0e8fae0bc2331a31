"""Data augmentation (the reference's ``augmentation.py``): token-level (masking, random replacement, span deletion,
sequence packing) and image-level (flip, crop, mixup, cutmix) transforms on torch tensors, all seeded."""
from __future__ import annotations

import torch


def mask_tokens(ids, mask_id, prob=0.15, generator=None, special=()):
    """BERT-style masking: returns (masked ids, labels with -100 where not selected)."""
    sel = torch.rand(ids.shape, generator=generator, device=ids.device) < prob
    for s in special:
        sel &= ids != s
    labels = torch.where(sel, ids, torch.full_like(ids, -100))
    return torch.where(sel, torch.full_like(ids, mask_id), ids), labels


def random_replace(ids, vocab_size, prob=0.05, generator=None):
    sel = torch.rand(ids.shape, generator=generator, device=ids.device) < prob
    rnd = torch.randint(0, vocab_size, ids.shape, generator=generator, device=ids.device)
    return torch.where(sel, rnd, ids)


def delete_span(ids, max_len=5, pad_id=0, generator=None):
    """Deletes one random span per row and pads at the end."""
    B, S = ids.shape
    out = ids.clone()
    for b in range(B):
        n = int(torch.randint(1, max_len + 1, (1,), generator=generator))
        s = int(torch.randint(0, max(1, S - n), (1,), generator=generator))
        out[b] = torch.cat([ids[b, :s], ids[b, s + n:], ids.new_full((n,), pad_id)])
    return out


def pack_sequences(seqs, seq_len, pad_id=0, eos_id=None):
    """Greedy packing of variable-length token lists into rows of ``seq_len`` (documents separated by ``eos_id``)."""
    rows, cur = [], []
    for s in seqs:
        s = list(s) + ([eos_id] if eos_id is not None else [])
        while s:
            room = seq_len - len(cur)
            cur += s[:room]
            s = s[room:]
            if len(cur) == seq_len:
                rows.append(cur)
                cur = []
    if cur:
        rows.append(cur + [pad_id] * (seq_len - len(cur)))
    return torch.tensor(rows, dtype=torch.long)


def random_flip(img, prob=0.5, generator=None):
    flip = torch.rand(img.shape[0], generator=generator, device=img.device) < prob
    return torch.where(flip[:, None, None, None], img.flip(-1), img)


def random_crop(img, size, padding=0, generator=None):
    if padding:
        img = torch.nn.functional.pad(img, (padding,) * 4)
    B, _, H, W = img.shape
    ys = torch.randint(0, H - size + 1, (B,), generator=generator)
    xs = torch.randint(0, W - size + 1, (B,), generator=generator)
    return torch.stack([img[b, :, ys[b]: ys[b] + size, xs[b]: xs[b] + size] for b in range(B)])


def mixup(x, y_onehot, alpha=0.2, generator=None):
    lam = float(torch.distributions.Beta(alpha, alpha).sample()) if alpha > 0 else 1.0
    perm = torch.randperm(x.shape[0], generator=generator, device=x.device)
    return lam * x + (1 - lam) * x[perm], lam * y_onehot + (1 - lam) * y_onehot[perm]


def cutmix(x, y_onehot, alpha=1.0, generator=None):
    lam = float(torch.distributions.Beta(alpha, alpha).sample())
    B, _, H, W = x.shape
    perm = torch.randperm(B, generator=generator, device=x.device)
    rh, rw = int(H * (1 - lam) ** 0.5), int(W * (1 - lam) ** 0.5)
    cy, cx = int(torch.randint(0, H, (1,), generator=generator)), int(torch.randint(0, W, (1,), generator=generator))
    y0, y1, x0, x1 = max(cy - rh // 2, 0), min(cy + rh // 2, H), max(cx - rw // 2, 0), min(cx + rw // 2, W)
    out = x.clone()
    out[:, :, y0:y1, x0:x1] = x[perm][:, :, y0:y1, x0:x1]
    lam_eff = 1 - (y1 - y0) * (x1 - x0) / (H * W)
    return out, lam_eff * y_onehot + (1 - lam_eff) * y_onehot[perm]
