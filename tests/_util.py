"""Helpers shared by the parity tests."""
import torch


def close_1e6(actual: torch.Tensor, ref64: torch.Tensor, rtol: float = 1e-6):
    """|actual - ref| <= rtol * max(|ref|, rms(ref)), element-wise, against a double-precision reference.

    The floor is needed because an fp32 array cannot hold elements near zero to 1e-6 of their own
    magnitude after a cancelling update; it ties the bound to the tensor's typical magnitude.
    Returns (ok, worst ratio of error to bound).
    """
    a = actual.detach().double().cpu()
    r = ref64.detach().double().cpu()
    nan_a, nan_r = torch.isnan(a), torch.isnan(r)
    if not torch.equal(nan_a, nan_r):
        return False, float('inf')
    a = torch.where(nan_a, torch.zeros_like(a), a)
    r = torch.where(nan_r, torch.zeros_like(r), r)
    finite = torch.isfinite(r)
    if not torch.equal(a[~finite], r[~finite]):
        return False, float('inf')
    a, r = a[finite], r[finite]
    if r.numel() == 0:
        return True, 0.0
    rms = r.pow(2).mean().sqrt()
    bound = rtol * torch.maximum(r.abs(), rms.expand_as(r))
    bound = torch.clamp(bound, min=1e-45)
    ratio = ((a - r).abs() / bound).max().item()
    return ratio <= 1.0, ratio


def lowp_within_1ulp(got: torch.Tensor, want: torch.Tensor, master_ref: torch.Tensor):
    """Working copies agree within 1 unit in the last place of the 16-bit format.

    `want` is the oracle's rounded master, `got` the kernel's; the two masters may differ by the fp32
    bound of :func:`close_1e6`, so the test is |got - want| <= spacing(want) + 1e-6 * max(|ref|, rms(ref)).
    (A plain integer ulp distance is meaningless for bf16 values near zero, whose spacing is far below
    the fp32 rounding error of the master.)  Returns (ok, worst ratio).
    """
    assert got.dtype == want.dtype and got.dtype in (torch.float16, torch.bfloat16)
    g = got.detach().cpu().double()
    w = want.detach().cpu().double()
    r = master_ref.detach().cpu().double()
    nan_g, nan_w = torch.isnan(g), torch.isnan(w)
    if not torch.equal(nan_g, nan_w):
        return False, float('inf')
    inf_w = torch.isinf(w)
    if not torch.equal(g[inf_w], w[inf_w]):
        return False, float('inf')
    keep = ~(nan_w | inf_w)
    g, w, r = g[keep], w[keep], r[keep]
    if w.numel() == 0:
        return True, 0.0
    mant_bits, min_exp = (10, -14) if got.dtype == torch.float16 else (7, -126)
    exp = torch.floor(torch.log2(torch.clamp(w.abs(), min=2.0**min_exp)))
    spacing = torch.pow(torch.tensor(2.0, dtype=torch.float64), exp - mant_bits)
    finite_r = r[torch.isfinite(r)]
    rms = finite_r.pow(2).mean().sqrt() if finite_r.numel() else torch.tensor(0.0, dtype=torch.float64)
    bound = spacing + 1e-6 * torch.maximum(r.abs(), rms.expand_as(r))
    ratio = ((g - w).abs() / bound).max().item()
    return ratio <= 1.0, ratio


def bits_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    a, b = a.detach().cpu().contiguous(), b.detach().cpu().contiguous()
    if a.dtype != b.dtype or a.shape != b.shape:
        return False
    view = {2: torch.int16, 4: torch.int32, 8: torch.int64}[a.element_size()]
    return torch.equal(a.view(view), b.view(view))


def make_chunk(n, dtype, seed, scale=64.0, sigma=1e-3, device='cpu'):
    """Seeded synthetic shard: master ~ N(0, 0.02), grads = (N(0, sigma) * scale) in `dtype`, zero moments."""
    gen = torch.Generator(device='cpu').manual_seed(seed)
    master = torch.randn(n, generator=gen) * 0.02
    grad = (torch.randn(n, generator=gen) * sigma * scale).to(dtype)
    return (master.to(device), torch.zeros(n, device=device), torch.zeros(n, device=device), grad.to(device))


def free_port() -> int:
    """A TCP port on 127.0.0.1 that nobody listens on right now (for a rendezvous of child processes)."""
    import socket
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]
