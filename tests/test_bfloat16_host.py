"""Host-side bfloat16 helpers (cudanative.jl_b200/bfloat16.py): rounding to nearest even, exact
widening, and the element-type tags the GEMM entry points take.  No GPU needed."""
import numpy as np
import pytest
import torch

from cudanative_jl_b200 import _lib
from cudanative_jl_b200.bfloat16 import BFloat16, round_to_bf16, widen_bf16


def test_round_to_nearest_even_known_answers():
    # value                         -> bits     why
    cases = [(0.0, 0x0000), (-0.0, 0x8000), (1.0, 0x3F80), (-2.0, 0xC000),
             (1.00390625, 0x3F80),            # 1 + 2^-8: exactly half way, tie goes to the even pattern below
             (1.01171875, 0x3F82),            # 1 + 3 * 2^-8: half way, tie goes up to the even pattern
             (1.0078125 + 2.0 ** -9, 0x3F81),  # just above a representable value: rounds down to it
             (3.3895314e38, 0x7F7F),          # largest finite bfloat16
             (3.4e38, 0x7F80),                # beyond it: overflows to infinity as IEEE rounding does
             (np.inf, 0x7F80), (-np.inf, 0xFF80),
             (1e-40, 0x0001)]                 # binary32 subnormal -> bfloat16 subnormal
    x = np.array([c[0] for c in cases], dtype=np.float32)
    assert [int(b) for b in round_to_bf16(x)] == [c[1] for c in cases]
    nan = round_to_bf16(np.array([np.nan], dtype=np.float32))
    assert np.isnan(widen_bf16(nan))[0]


@pytest.mark.parametrize("order", ["C", "F"])
def test_round_and_widen_match_torch(order):
    x = (np.random.default_rng(7).standard_normal((53, 17)) * 10.0 ** np.random.default_rng(8).integers(-20, 20, (53, 17))).astype(np.float32)
    x = np.asarray(x, order=order)
    bits = round_to_bf16(x)
    assert bits.dtype == np.uint16 and bits.shape == x.shape
    want = torch.from_numpy(np.ascontiguousarray(x)).to(torch.bfloat16)
    assert np.array_equal(bits, want.view(torch.int16).numpy().view(np.uint16))
    assert np.array_equal(widen_bf16(bits), want.float().numpy())
    # keeps the memory order of its input, so a Fortran matrix stays a Fortran matrix
    assert bits.flags.f_contiguous == x.flags.f_contiguous
    # idempotent: a bfloat16 value survives widening and rounding unchanged
    assert np.array_equal(round_to_bf16(widen_bf16(bits)), bits)


def test_type_tags():
    from cudanative_jl_b200.gemm import _type_code

    assert _type_code(np.float16) == _lib.F16 == 0
    assert _type_code(np.float32) == _lib.F32 == 1
    assert _type_code(BFloat16) == _lib.BF16 == 2
    with pytest.raises(TypeError):
        _type_code(np.float64)


def test_library_helpers_agree_with_the_oracle(oracle):
    """The oracle rounds by comparing the dropped bits with the half-way point, the library's helper by
    add-and-shift: two statements of round-to-nearest-even that must give the same bits."""
    rand = np.random.default_rng(11)
    x = (rand.standard_normal(20000) * 10.0 ** rand.integers(-30, 30, 20000)).astype(np.float32)
    ties = (np.arange(0x3F80, 0x3F80 + 512, dtype=np.uint32) << 16 | 0x8000).view(np.float32)  # exact half-way cases
    special = np.array([0.0, -0.0, np.inf, -np.inf, 3.3895314e38, 3.4e38, -3.4e38, 1e-40, -1e-45], dtype=np.float32)
    for arr in (x, ties, special, np.asfortranarray(x[:600].reshape(20, 30))):
        assert np.array_equal(round_to_bf16(arr), oracle.bf16_round(arr))
        bits = oracle.bf16_round(arr)
        assert np.array_equal(widen_bf16(bits), oracle.bf16_widen(bits))
    nan = oracle.bf16_round(np.array([np.nan, -np.nan], dtype=np.float32))
    assert np.all(np.isnan(oracle.bf16_widen(nan)))
