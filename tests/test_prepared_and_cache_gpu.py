"""Per-call host cost: a prepared product (argument structures built once) gives the same result
as the convenience wrapper, and the tensor maps of a product that comes back with the same views
are taken from the cache instead of being encoded again."""
import numpy as np
import pytest
import torch

from gpu_util import dev, host, rel_to_max

pytestmark = pytest.mark.gpu


def test_prepared_call_equals_wrapper_and_follows_new_values(ttb):
    rng = np.random.default_rng(120)
    a = rng.standard_normal((3, 200, 96)).astype(np.float32)
    bt = rng.standard_normal((3, 136, 96)).astype(np.float32)
    A, Bt = dev(a), dev(bt)
    out = torch.zeros((3, 200, 136), device="cuda")
    pm = ttb.PreparedMatmul(A, Bt.permute(0, 2, 1), out)
    assert pm() is out
    assert torch.equal(out, ttb.batched_matmul(A, Bt.permute(0, 2, 1)))
    a2 = rng.standard_normal(a.shape).astype(np.float32)
    A.copy_(dev(a2))                      # same buffers, new values: the prepared call reads them
    pm()
    want = np.matmul(a2.astype(np.float64), bt.astype(np.float64).transpose(0, 2, 1))
    assert rel_to_max(host(out), want) <= 1e-5
    with pytest.raises(ttb.TTBError):
        ttb.PreparedMatmul(A, Bt, out)    # inner dims do not match the result shape
    ttb.check_device(0)


def test_repeated_views_hit_the_tensor_map_cache(ttb):
    A = torch.randn((2, 256, 128), device="cuda")
    B = torch.randn((2, 128, 256), device="cuda")
    out = torch.empty((2, 256, 256), device="cuda")
    ttb.batched_matmul(A, B, out=out)                       # encodes (or finds) lhs, rhs and result maps
    assert ttb.last_variant() in (ttb.Variant.TCGEN05_3XTF32, ttb.Variant.TCGEN05_2CTA)
    h0, m0 = ttb.tensor_map_cache_stats()
    for _ in range(5):
        ttb.batched_matmul(A, B, out=out)
    h1, m1 = ttb.tensor_map_cache_stats()
    assert m1 == m0 and h1 - h0 == 15                       # three maps per call, all from the cache
    # another view of the same storage is another key
    ttb.batched_matmul(A[:, :128], B, out=out[:, :128])
    h2, m2 = ttb.tensor_map_cache_stats()
    assert m2 - m1 >= 2
    want = torch.matmul(A.double(), B.double())
    assert float((out.double() - want).abs().max() / want.abs().max()) <= 1e-5
