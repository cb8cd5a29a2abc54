"""tcgen05 batched A.B^T against an fp32 matmul of the same bf16 operands."""
import pytest
import torch

from gpu_util import assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("batch,M,N,K", [
    (1, 128, 128, 64),      # one tile, one K slab
    (3, 128, 128, 256),     # batching, K loop
    (2, 256, 384, 192),     # several tiles, BN=128
    (1, 384, 512, 1024),    # BN=256 path, ring wraps
    (2, 100, 72, 40),       # ragged M/N/K: TMA zero fill and store bounds
    (130, 128, 256, 128),   # more tiles than CTAs can hold at once for one wave of channels
])
def test_bmm_nt(batch, M, N, K):
    from bioemu2_b200 import functional as F

    g = torch.Generator(device="cuda").manual_seed(batch * 1000 + M + N + K)
    a = torch.randn(batch, M, K, device="cuda", generator=g).bfloat16()
    b = torch.randn(batch, N, K, device="cuda", generator=g).bfloat16()
    c = F.bmm_nt(a, b, scale=0.5)
    ref = 0.5 * torch.matmul(a.double(), b.double().transpose(1, 2))
    assert_close(f"bmm_nt[{batch},{M},{N},{K}]", c, ref, rel=5e-3)  # only the bf16 rounding of the output


def test_layernorm_rows():
    from bioemu2_b200 import functional as F

    g = torch.Generator(device="cuda").manual_seed(3)
    for cols in (64, 128, 384, 768):
        x = (torch.randn(1000, cols, device="cuda", generator=g) * 3 + 1).bfloat16()
        w = torch.randn(cols, device="cuda", generator=g)
        b = torch.randn(cols, device="cuda", generator=g)
        y = F.layernorm(x, w, b)
        ref = torch.nn.functional.layer_norm(x.double(), (cols,), w.double(), b.double())
        assert_close(f"layernorm[{cols}]", y, ref, rel=5e-3)


def test_linear_bias_is_not_read_past_its_end():
    """out_features = 160 is a multiple of 32 but not of the 128-column output tile: the last column tile of the bulk
    epilogue must not read bias entries beyond the 160th.  The bias sits at the very end of its allocation and the
    columns beyond it are poisoned, so an unguarded read would show up as NaN or as a fault."""
    from bioemu2_b200 import functional as F

    g = torch.Generator().manual_seed(5)
    rows, fin, fout = 256, 64, 160
    x = torch.randn(rows, fin, generator=g)
    w = torch.randn(fout, fin, generator=g) / 8
    store = torch.full((4096,), float("nan"))
    store[-fout:] = torch.randn(fout, generator=g)
    bias = store.cuda()[-fout:]
    for out_dtype in (torch.float32, torch.bfloat16):
        out = F.linear_bf16(x.bfloat16().cuda(), w.bfloat16().cuda(), bias, out_dtype=out_dtype)
        ref = x.bfloat16().double() @ w.bfloat16().double().T + store[-fout:].double()
        assert_close(f"linear_out160_bias_{out_dtype}", out, ref)
