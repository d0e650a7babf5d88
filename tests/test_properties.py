"""Property tests (hypothesis) of the quantiser, the wire formats and the compatibility packers."""
import numpy as np
import torch
from hypothesis import given, settings, strategies as st

from gradient_compression_b200 import ops
from gradient_compression_b200.ops import packing

BITS = st.sampled_from([1, 2, 3, 4, 6, 8, 10, 12])


@settings(max_examples=60, deadline=None)
@given(bits=BITS, n=st.integers(1, 3000), seed=st.integers(0, 2**31 - 1), scale=st.floats(1e-6, 1e6))
def test_levels_stay_in_range_and_within_one_step(bits, n, seed, scale):
    """|level| <= s, sign(level) = sign(x) (or 0), and the dequantised value is within one quantisation step of x."""
    s = (1 << bits) - 1
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(n, generator=g) * scale).float()
    norm = float(x.abs().max())
    q = ops.quantize_levels(x, norm, s, seed=seed, stream=3, step=seed % 17)
    assert int(q.abs().max()) <= s
    assert bool(((q == 0) | (torch.sign(q.float()) == torch.sign(x))).all())
    y = ops.dequantize_levels(q, norm, s)
    assert float((y - x).abs().max()) <= norm / s * (1 + 1e-5) + 1e-30


@settings(max_examples=60, deadline=None)
@given(bits=BITS, n=st.integers(1, 3000), seed=st.integers(0, 2**31 - 1))
def test_wire_format_round_trip(bits, n, seed):
    s = (1 << bits) - 1
    g = torch.Generator().manual_seed(seed)
    q = torch.randint(-s, s + 1, (n,), generator=g, dtype=torch.int32)
    mags, signs = ops.pack_levels(q, bits)
    mag_bytes, sign_bytes = ops.packed_sizes(n, bits)
    assert mags.numel() * mags.element_size() == mag_bytes and signs.numel() * signs.element_size() == sign_bytes
    assert torch.equal(ops.unpack_levels(mags, signs, n, bits), q)


@settings(max_examples=40, deadline=None)
@given(s=st.integers(1, 65535), world=st.integers(1, 8))
def test_sum_container_holds_every_possible_sum(s, world):
    """W ranks of levels in [-s, s] sum to at most W s in magnitude: the container chosen for the summed levels holds it."""
    dt = ops.sum_container_dtype(s, world)
    assert torch.iinfo(dt).max >= s * world and torch.iinfo(dt).min <= -s * world


@settings(max_examples=60, deadline=None)
@given(vals=st.lists(st.integers(0, 255), min_size=1, max_size=400))
def test_variable_width_packer_round_trip_and_is_never_larger_than_bytes(vals):
    src = torch.tensor(vals, dtype=torch.int32)
    words = packing.varpack(src)
    assert torch.equal(packing.varunpack(words, len(vals)), src)
    assert words.numel() <= (len(vals) + 2) // 3            # worst case: three 8-bit values per 32-bit word


@settings(max_examples=60, deadline=None)
@given(vals=st.lists(st.integers(-128, 127), min_size=1, max_size=300))
def test_byte_packer_round_trip(vals):
    src = torch.tensor(vals, dtype=torch.int32)
    assert torch.equal(packing.byteunpack(packing.bytepack(src), len(vals)).to(torch.int32), src)


@settings(max_examples=60, deadline=None)
@given(vals=st.lists(st.integers(-255, 255), min_size=1, max_size=200), norm=st.floats(1e-3, 1e3))
def test_elias_stream_round_trip(vals, norm):
    q = torch.tensor(vals, dtype=torch.int32)
    got_norm, got = packing.elias_decode(packing.elias_encode(q, norm))
    assert torch.equal(got[:len(vals)], q) and abs(got_norm - np.float32(norm)) <= 1e-6 * abs(norm)
