"""The allocation-free triangle multiplication entry point against the workspace one.

Some embedders of the library cannot give it a workspace: their device memory belongs to another
framework's pool, or they run where a cudaMalloc (and the device-wide synchronisation it implies) is not
allowed.  ``b200_trimul_fwd_static`` serves them from a fixed scratch array inside the library.  This test
calls both entry points through the C ABI on the same inputs, twice in a row (the second call reuses
whatever the first left in the scratch), and expects identical results; before that it fills the scratch with
NaN through a full-size call, because the padded rows and columns of the scratch planes are not rewritten by a
smaller call and must not reach its output.  It also checks the size limit.
Collected last on purpose, so a run that stops at the first failure has already seen every other test.
"""
import ctypes

import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu


def _call(fn, z, mask, out, packed, N, incoming, *extra):
    import bioemu2_b200._lib as L

    stream = torch.cuda.current_stream().cuda_stream
    return fn(z.data_ptr(), mask.data_ptr(), out.data_ptr(), ctypes.byref(packed.struct), 1, N, incoming, 0,
              L.DTYPE_F32, *extra, stream)


@pytest.mark.parametrize("N", [96, 200])
def test_static_scratch_matches_workspace_entry_point(N):
    import bioemu2_b200._lib as L
    from bioemu2_b200 import functional as F

    lib = L.lib
    g = torch.Generator().manual_seed(900 + N)
    w = H.trimul_weights(g)
    packed = F.TriMulPacked(*[w[k].cuda() for k in ("norm_in.weight", "norm_in.bias", "p_in.weight", "g_in.weight",
                                                     "norm_out.weight", "norm_out.bias", "p_out.weight", "g_out.weight")])
    nbytes = lib.b200_trimul_workspace_bytes(N)
    ws = F.workspace(nbytes, torch.device("cuda", torch.cuda.current_device()))
    # hostile leftovers: a call at the size limit on an all-NaN pair tensor leaves NaN in every plane of the scratch
    zn = torch.full((1, 256, 256, 128), float("nan"), device="cuda")
    mn = torch.ones(1, 256, 256, dtype=torch.uint8, device="cuda")
    L.check(_call(lib.b200_trimul_fwd_static, zn, mn, torch.empty_like(zn), packed, 256, 0))
    torch.cuda.synchronize()
    for call in range(2):  # two calls in a row: the second sees the first one's leftovers in the scratch
        z = torch.randn(1, N, N, 128, generator=g).cuda()
        mask = (torch.rand(1, N, N, generator=g) > 0.25).to(torch.uint8).cuda()
        for incoming in (0, 1):
            ref = torch.empty_like(z)
            got = torch.full_like(z, float("nan"))
            L.check(_call(lib.b200_trimul_fwd, z, mask, ref, packed, N, incoming, ws.data_ptr(), nbytes))
            L.check(_call(lib.b200_trimul_fwd_static, z, mask, got, packed, N, incoming))
            torch.cuda.synchronize()
            assert L.device_status() == 0
            assert not torch.isnan(got).any(), "stale scratch contents reached the output"
            # same kernels, same inputs: the tolerance of the other parity tests (2e-2 of max) is far from needed
            torch.testing.assert_close(got, ref, atol=1e-6, rtol=0, msg=f"call {call}, incoming={incoming}")


def test_static_scratch_rejects_sizes_beyond_its_limit():
    import bioemu2_b200._lib as L
    from bioemu2_b200 import functional as F

    g = torch.Generator().manual_seed(1)
    w = H.trimul_weights(g)
    packed = F.TriMulPacked(*[w[k].cuda() for k in ("norm_in.weight", "norm_in.bias", "p_in.weight", "g_in.weight",
                                                     "norm_out.weight", "norm_out.bias", "p_out.weight", "g_out.weight")])
    N = 257
    z = torch.zeros(1, N, N, 128, device="cuda")
    mask = torch.ones(1, N, N, dtype=torch.uint8, device="cuda")
    out = torch.empty_like(z)
    status = _call(L.lib.b200_trimul_fwd_static, z, mask, out, packed, N, 0)
    assert status == L.ERR_INVALID_ARGUMENT
    assert "256" in L.last_error()
