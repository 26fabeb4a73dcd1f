"""The AVX2/F16C kernels of the host data path against the scalar software
conversions (which PyTorch's own fp16/bf16 arithmetic confirms): sum, scale,
Adasum dot/norms and scaled add, on lengths around the vector width and on
special values (subnormals, infinities, NaN, rounding ties)."""
import numpy as np
import pytest
import torch

from horovod_b200 import _C

T = _C.testing
F16, BF16 = 6, 10
SUM = 1


def _bits(t):
    return t.view(torch.int16).numpy().tobytes()


def _from_bits(raw, dtype):
    return torch.frombuffer(bytearray(raw), dtype=torch.int16).view(dtype)


def _samples(n, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, generator=g) * torch.logspace(-8, 4, n)
    special = torch.tensor([0.0, -0.0, float("inf"), float("-inf"), float("nan"), 65504.0,
                            6e-8, -6e-8, 1.0009765625, 2049.0, 3.3895314e38])
    k = min(n, special.numel())
    x[:k] = special[:k]
    return x.to(dtype)


@pytest.mark.parametrize("dtype,code", [(torch.float16, F16), (torch.bfloat16, BF16)])
@pytest.mark.parametrize("n", [1, 7, 8, 9, 16, 31, 1000, 4099])
def test_vector_and_scalar_paths_agree_bit_for_bit(dtype, code, n):
    a, b = _samples(n, dtype, 1), _samples(n, dtype, 2).flip(0)
    results = {}
    for scalar in (True, False):
        T.cpu_vector_force_scalar(scalar)
        try:
            s = T.reduce_into(_bits(a), _bits(b), n, code, SUM)
            m = T.scale_buffer(_bits(a), n, code, 0.3)
            d = T.dot_norms_16(_bits(a), _bits(b), dtype == torch.float16)
            c = T.scaled_add_16(_bits(a), _bits(b), 0.75, -1.25, dtype == torch.float16)
        finally:
            T.cpu_vector_force_scalar(False)
        results[scalar] = (s, m, d, c)
    if not T.cpu_has_f16c():
        pytest.skip("this CPU has no AVX2 + F16C: only the scalar path exists")
    sv, ss = results[False], results[True]
    assert sv[0] == ss[0], "sum differs"
    assert sv[1] == ss[1], "scale differs"
    assert sv[3] == ss[3], "scaled add differs"
    for x, y in zip(sv[2], ss[2]):  # accumulation order differs: compare numerically
        assert (np.isnan(x) and np.isnan(y)) or x == pytest.approx(y, rel=1e-12) or \
            (np.isinf(x) and x == y)


@pytest.mark.parametrize("dtype,code", [(torch.float16, F16), (torch.bfloat16, BF16)])
def test_sum_and_scale_match_pytorch(dtype, code):
    n = 1003
    g = torch.Generator().manual_seed(5)
    a = torch.randn(n, generator=g).to(dtype)
    b = torch.randn(n, generator=g).to(dtype)
    got = _from_bits(T.reduce_into(_bits(a), _bits(b), n, code, SUM), dtype)
    assert torch.equal(got, (a.float() + b.float()).to(dtype))
    got = _from_bits(T.scale_buffer(_bits(a), n, code, 0.3), dtype)
    assert torch.equal(got, (a.float() * torch.tensor(0.3)).to(dtype))
    dot, na, nb = T.dot_norms_16(_bits(a), _bits(b), dtype == torch.float16)
    assert dot == pytest.approx(float(a.double() @ b.double()), rel=1e-12)
    assert na == pytest.approx(float(a.double() @ a.double()), rel=1e-12)
    assert nb == pytest.approx(float(b.double() @ b.double()), rel=1e-12)
    got = _from_bits(T.scaled_add_16(_bits(a), _bits(b), 0.75, -1.25,
                                     dtype == torch.float16), dtype)
    assert torch.equal(got, (0.75 * a.double() - 1.25 * b.double()).float().to(dtype))
