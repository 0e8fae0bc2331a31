"""Self-supervised pre-training of a small masked autoencoder on synthetic images, then reconstruction of one image
from a quarter of its patches."""
from _common import device, seed  # first: makes the package importable from a checkout
import torch

from sneppx.models.families import MAE
from sneppx.optim.zoo import AdamW


def main(steps: int = 150) -> float:
    g, dev = seed(4), device()
    yy, xx = torch.meshgrid(torch.linspace(-1, 1, 32), torch.linspace(-1, 1, 32), indexing="ij")
    phase = torch.rand(64, 1, 1, generator=g) * 6.28
    imgs = torch.stack([torch.sin(4 * xx + phase), torch.cos(4 * yy + phase), torch.sin(3 * (xx + yy) + phase)], 1).to(dev)
    model = MAE(img_size=32, patch_size=8, embed_dim=64, encoder_depth=2, decoder_depth=1, num_heads=4, decoder_embed_dim=32,
                mask_ratio=0.75, device=dev)
    opt = AdamW(model.parameters(), lr=3e-3, weight_decay=0.05)
    fixed = torch.rand(64, 16, generator=g).to(dev)            # one masking pattern to compare before / after on
    with torch.no_grad():
        before = model(imgs, noise=fixed)[0].item()
    for _ in range(steps):
        opt.zero_grad()
        loss, _, _ = model(imgs)                               # a fresh random mask every step
        loss.backward()
        opt.step()
    with torch.no_grad():
        after, pred, mask = model(imgs, noise=fixed)
        recon = model.unpatchify(pred)
    print(f"masked-patch MSE {before:.3f} -> {after.item():.3f}; reconstructed {tuple(recon.shape)} from "
          f"{int((1 - mask[0]).sum())} of {mask.shape[1]} patches per image")
    return after.item() / before


if __name__ == "__main__":
    main()
