"""Plain PyTorch FP32 restatement of the device quantizer, shared by the single-GPU kernel tests and the
multi-GPU worker."""
import torch


def bf16_ceil(x: torch.Tensor) -> torch.Tensor:
    """Smallest bf16 >= x for x >= 0 (as float32)."""
    b = x.float().view(torch.int32)
    b = ((b + 0xFFFF) >> 16) << 16
    return b.view(torch.float32)


def ref_quantize(e: torch.Tensor):
    """Block-64 INT4, round to nearest: scale = bf16_ceil(amax * fl32(1/7)), q = floor(e / scale + 0.5)
    clamped to [-8, 7]. Returns (dequantized values, per-block scales)."""
    n = e.numel()
    pad = (-n) % 64
    x = torch.cat([e.float(), e.new_zeros(pad, dtype=torch.float32)]).view(-1, 64)
    amax = x.abs().amax(dim=1, keepdim=True)
    s = bf16_ceil(amax * 0.14285715)
    live = s > 1e-30
    inv = torch.where(live, 1.0 / s, torch.zeros_like(s))
    q = torch.floor(x * inv + 0.5).clamp_(-8, 7)
    deq = torch.where(live, q * s, torch.zeros_like(q))
    return deq.view(-1)[:n], s.view(-1)
