"""The allocation-free prefill entry point against the regular one (runs last: its file sorts last).

Who needs it: hosts that may not touch the CUDA allocator at the moment they run a prefill, e.g. a
serving loop inside an allocation-free critical section or a process whose device memory belongs to
another runtime's pool.  The regular b200q_dense takes a stream-ordered buffer for the bf16 copy of
f32 activations; b200q_dense_f32_prefill_noalloc keeps that copy in a fixed 8 MiB array of the library.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import gomlx_b200 as g  # noqa: E402
from gomlx_b200 import _native as nat  # noqa: E402
from gomlx_b200.quantize import synthetic_weights  # noqa: E402


def _noalloc(wr, x, bias, act, y):
    return nat.lib().b200q_dense_f32_prefill_noalloc(
        wr.handle, ctypes.c_void_p(x.data_ptr()), x.shape[0], ctypes.c_void_p(bias.data_ptr()) if bias is not None else None,
        int(act), ctypes.c_void_p(y.data_ptr()), 0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("name", ["Q4_K", "Q8_0"])
def test_noalloc_matches_regular_entry_point_twice(name):
    t = g.GGMLQuantType[name]
    n, k = 300, 1280
    wr = g.upload(synthetic_weights(t, n, k, seed=4), t)
    quant = g.Quantization(g.QuantizationScheme.GGML, t)
    gen = torch.Generator(device="cuda").manual_seed(7)
    bias = torch.randn(n, device="cuda", generator=gen)
    for m in (200, 64):  # two calls in a row share the static array; the second is smaller than the first
        x = torch.randn(m, k, device="cuda", generator=gen)
        want = g.backend_fused_quantized_dense(x, wr, bias, quant, g.ActivationType.SILU)
        got = torch.full((m, n), float("nan"), device="cuda")
        assert _noalloc(wr, x, bias, g.ActivationType.SILU, got) == nat.OK, nat.lib().b200q_last_error()
        torch.cuda.synchronize()
        assert nat.lib().b200q_weight_check(wr.handle, None) == nat.OK
        # same kernels on the same bf16 values: the tolerance of the GEMM tests (1e-2) is far from needed
        err = float((got - want).abs().max() / want.abs().max())
        assert err <= 1e-6, err
    wr.free()


def test_noalloc_rejects_oversize_and_decode_shapes():
    t = g.GGMLQuantType.Q4_K
    cap = nat.lib().b200q_noalloc_capacity()
    assert cap == 4 * 1024 * 1024
    k = 4096
    wr = g.upload(synthetic_weights(t, 32, k, seed=1), t)
    m = cap // k + 1  # one row too many
    x = torch.zeros(m, k, device="cuda")
    y = torch.zeros(m, 32, device="cuda")
    assert _noalloc(wr, x, None, g.ActivationType.NONE, y) == nat.EINVAL
    assert b"exceeds" in nat.lib().b200q_last_error()
    assert _noalloc(wr, x[:8], None, g.ActivationType.NONE, y[:8]) == nat.EINVAL  # decode sizes take b200q_dense
    assert _noalloc(wr, x[:cap // k], None, g.ActivationType.NONE, y[:cap // k]) == nat.OK  # exactly at the limit
    torch.cuda.synchronize()
    assert float(y.abs().max()) == 0.0
    wr.free()
