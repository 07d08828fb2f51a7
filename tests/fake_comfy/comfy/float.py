import torch


def stochastic_rounding(x: torch.Tensor, dtype: torch.dtype, seed: int | None = None) -> torch.Tensor:
    """Test double: ComfyUI's real implementation is external.  Rounds x to `dtype` stochastically with a seeded
    generator (unbiased between the two neighbouring representable values).  Only its contract matters to the tests:
    the result has dtype `dtype`, the same shape, and every element is one of the two neighbours of x."""
    if dtype != torch.float8_e5m2:
        return x.to(dtype)
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed or 0))
    xf = x.detach().to("cpu", torch.float32)
    lo = xf.to(dtype).to(torch.float32)
    # neighbour on the other side of x
    bits = lo.to(dtype).view(torch.uint8).to(torch.int16)
    step = torch.where(xf.abs() > lo.abs(), 1, -1).to(torch.int16)
    other = ((bits + step).clamp(0, 255)).to(torch.uint8).view(dtype).to(torch.float32)
    span = (other - lo).abs().clamp_min(1e-30)
    p_other = ((xf - lo).abs() / span).clamp(0, 1)
    p_other = torch.where(torch.isfinite(p_other), p_other, torch.zeros_like(p_other))
    take_other = torch.rand(xf.shape, generator=gen) < p_other
    out = torch.where(take_other & (xf != lo), other, lo)
    return out.to(dtype).to(x.device)
