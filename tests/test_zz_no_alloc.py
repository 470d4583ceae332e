"""The allocation-free bias gradient (vtlb_bias_grad_f32_noalloc).

It exists for hosts that cannot let the library allocate on the device while they run -
all of HBM already belongs to their own pools, or an allocation's implicit synchronisation
would break their latency budget - so its partial sums live in a fixed array inside the
library instead of the context's scratch.  Checked here: it gives what the allocating entry
point (vtlb_linear_bwd_f32 asked for db only) gives, on two calls in a row that share the
array, and it refuses widths beyond the array's fixed size.  This file sorts last so that a
run that stops at the first failure has already run every other test."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _both(dev, G):
    M, N = G.shape
    dG = dev.to_device(G)
    ref, got = dev.zeros(N), dev.zeros(N)
    dev.linear_bwd_f32(dG, None, None, None, None, ref, M, N, 1)
    dev.bias_grad_f32_noalloc(dG, M, N, got)
    r, g = ref.numpy(), got.numpy()
    for b in (dG, ref, got):
        b.free()
    return r, g


def test_no_alloc_bias_grad_matches_allocating_entry_point_twice(dev):
    rng = np.random.default_rng(11)
    # two calls in a row; the second is narrower and shorter, so anything the first call
    # left in the shared array beyond the second call's extent must not leak into it
    for (M, N) in ((5000, 4096), (130, 70)):
        G = rng.standard_normal((M, N)).astype(np.float32)
        ref, got = _both(dev, G)
        tol = 1e-5 * np.sqrt(M) * float(np.abs(G).max())  # the bound the f32 tests use
        assert np.abs(got - ref).max() <= tol
        assert np.abs(got - G.astype(np.float64).sum(axis=0)).max() <= tol
    assert dev.check_status() == 0


def test_no_alloc_bias_grad_refuses_sizes_beyond_its_array(dev):
    from vtl_b200.capi import EINVAL, VtlbError
    G = dev.zeros((2, 4097))
    out = dev.zeros(4097)
    with pytest.raises(VtlbError) as e:
        dev.bias_grad_f32_noalloc(G, 2, 4097, out)
    assert e.value.code == EINVAL and "4096" in str(e.value)
    G.free(); out.free()
