"""CUDA quantize / pack / dequantize primitives against the reference's golden bytes and the oracle."""

import numpy as np
import pytest
import torch

import dartkv_b200 as dart
from dartkv_b200 import _lib
from dartkv_b200.quantization import _pack, _unpack
from oracle import dartkv_oracle as orc
from tests.helpers import TAG_DT, load_golden, to_np

pytestmark = pytest.mark.gpu

PRIM = load_golden("primitives.npz")
QUANT_KEYS = sorted({k.rsplit("/", 1)[0] for k in PRIM if k.startswith("quant/")})
MIXED_NAMES = sorted({k.split("/")[1] for k in PRIM if k.startswith("mixed/")})


def dev(array, dt):
    return torch.from_numpy(np.ascontiguousarray(array)).to(TAG_DT[dt]).cuda()


@pytest.mark.parametrize("key", QUANT_KEYS)
def test_quantize_is_bit_exact_against_reference(key):
    _, dt, bits, _ = key.split("/")
    axis, group, padded, packed = (int(v) for v in PRIM[f"{key}/meta"])
    md = str(PRIM[f"{key}/md"])
    data = dev(PRIM[f"{key}/input"], dt)
    q = dart.quantize(data, bits=int(bits[1:]), group_size=group, metadata_dtype=TAG_DT[md], axis=axis)
    assert (q.padded_dim, q.packed_dim, q.axis) == (padded, packed, axis % data.ndim)
    assert q.values.dtype == torch.uint8 and q.scale.dtype == TAG_DT[md]
    np.testing.assert_array_equal(to_np(q.values), PRIM[f"{key}/values"])
    np.testing.assert_array_equal(to_np(q.scale), PRIM[f"{key}/scale"])
    np.testing.assert_array_equal(to_np(q.zero_point), PRIM[f"{key}/zero"])
    restored = dart.dequantize(q)
    assert restored.dtype == data.dtype and restored.shape == data.shape
    np.testing.assert_array_equal(to_np(restored), PRIM[f"{key}/dequant"])
    # the fp32 single-rounding flavour agrees with the oracle's restatement of the reference's Triton kernels
    oq = orc.quantize(PRIM[f"{key}/input"], dt, bits=int(bits[1:]), group_size=group, md=md, axis=axis)
    np.testing.assert_array_equal(to_np(dart.triton_dequantize(q)), orc.dequantize(oq, flavour="fp32"))


@pytest.mark.parametrize("name", MIXED_NAMES)
@pytest.mark.parametrize("strategy", ["magnitude", "variance"])
def test_mixed_key_is_bit_exact_with_reference_channels(name, strategy):
    dt = str(PRIM[f"mixed/{name}/dt"])
    group = int(PRIM[f"mixed/{name}/group"])
    key = f"mixed/{name}/{strategy}"
    md = str(PRIM[f"{key}/md"])
    keys = dev(PRIM[f"mixed/{name}/input"], dt)
    ref_idx = torch.from_numpy(PRIM[f"{key}/indices"]).cuda()
    m = dart.quantize_key_mixed(keys, group_size=group, promote_ratio=0.25, metadata_dtype=TAG_DT[md],
                                strategy=strategy, indices=ref_idx)
    np.testing.assert_array_equal(to_np(m.low_values), PRIM[f"{key}/low"])
    np.testing.assert_array_equal(to_np(m.high_values), PRIM[f"{key}/high"])
    np.testing.assert_array_equal(to_np(m.channel_indices), PRIM[f"{key}/indices"])
    np.testing.assert_array_equal(to_np(m.scale), PRIM[f"{key}/scale"])
    np.testing.assert_array_equal(to_np(m.zero_point), PRIM[f"{key}/zero"])
    np.testing.assert_array_equal(to_np(m.dequantize()), PRIM[f"{key}/dequant"])
    assert m.promote_mask.sum().item() == ref_idx.numel()


@pytest.mark.parametrize("name", MIXED_NAMES)
@pytest.mark.parametrize("strategy", ["magnitude", "variance"])
def test_channel_selection_matches_oracle_rule(name, strategy):
    dt = str(PRIM[f"mixed/{name}/dt"])
    keys_np = PRIM[f"mixed/{name}/input"]
    keys = dev(keys_np, dt)
    scores = dart.channel_scores(keys, strategy=strategy)
    np.testing.assert_array_equal(to_np(scores), orc.channel_scores(keys_np, dt, strategy))
    mask, idx = dart.select_key_channels(keys, 0.25, strategy=strategy)
    omask, oidx = orc.select_key_channels(keys_np, dt, 0.25, strategy=strategy)
    np.testing.assert_array_equal(to_np(idx), oidx)
    np.testing.assert_array_equal(to_np(mask), omask)
    # and, through selection, the whole mixed page equals the oracle's
    group = int(PRIM[f"mixed/{name}/group"])
    m = dart.quantize_key_mixed(keys, group_size=group, promote_ratio=0.25, strategy=strategy)
    om = orc.quantize_key_mixed(keys_np, dt, group_size=group, ratio=0.25, strategy=strategy)
    np.testing.assert_array_equal(to_np(m.low_values), om.low_values)
    np.testing.assert_array_equal(to_np(m.high_values), om.high_values)
    np.testing.assert_array_equal(to_np(m.scale), om.scale)


def test_round_trip_error_bounds_and_shapes():
    # reference tests/test_quantization.py:7-23,37-59
    torch.manual_seed(1)
    source = torch.randn(2, 3, 7, dtype=torch.float32).cuda()
    for bits, tolerance in ((2, 0.55), (4, 0.12), (8, 0.01)):
        packed = dart.quantize(source, bits=bits, group_size=4, metadata_dtype=torch.float32)
        restored = dart.dequantize(packed)
        assert restored.shape == source.shape and restored.dtype == source.dtype
        assert torch.max(torch.abs(source - restored)).item() <= tolerance
        assert packed.nbytes < packed.dense_nbytes
    constant = torch.full((1, 5), 3.25, dtype=torch.float32).cuda()
    torch.testing.assert_close(dart.quantize(constant, bits=2, group_size=8, metadata_dtype=torch.float32).dequantize(),
                               constant)
    torch.manual_seed(3)
    source = torch.randn(2, 3, 9, 5).cuda()
    packed = dart.quantize_axis(source, axis=-2, bits=2, group_size=4, metadata_dtype=torch.float32)
    assert packed.scale.shape == (2, 3, 5, 3)
    assert torch.max((source - packed.dequantize()).abs()).item() < 0.9
    torch.manual_seed(4)
    source = torch.randn(1, 2, 17, 16).cuda()
    mask, indices = dart.select_key_channels(source, 0.25, strategy="magnitude")
    assert mask.shape == (1, 2, 16) and indices.shape == (1, 2, 4)
    mixed = dart.quantize_key_mixed(source, group_size=8, promote_ratio=0.25, metadata_dtype=torch.float32)
    assert mixed.high_values.shape[2] == 4 and mixed.promote_mask.sum().item() == 8
    assert mixed.nbytes < mixed.dense_nbytes
    assert torch.max((source - mixed.dequantize()).abs()).item() < 0.9


def test_nonfinite_input_is_rejected():
    with pytest.raises(ValueError, match="finite"):
        dart.quantize(torch.tensor([[float("nan")]]).cuda())
    with pytest.raises(ValueError, match="finite"):
        dart.quantize_key_mixed(torch.full((1, 1, 4, 4), float("inf")).cuda())


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_pack_unpack_round_trip(bits):
    rng = np.random.default_rng(bits)
    codes = rng.integers(0, 1 << bits, size=(5, 3, 37), dtype=np.uint8)
    vpb = 8 // bits
    packed_dim = -(-37 // vpb) * vpb
    packed = _pack(torch.from_numpy(codes).cuda(), bits, packed_dim)
    np.testing.assert_array_equal(to_np(packed), orc.pack_bits(codes, bits))
    np.testing.assert_array_equal(to_np(_unpack(packed, bits, 37)), codes)


def test_reciprocal_division_switch_matches_oracle():
    gen = torch.Generator().manual_seed(5)
    data = torch.randn(4, 256, generator=gen)
    for dt, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
        x = data.to(dt).cuda()
        q = dart.quantize(x, bits=2, group_size=32, division="reciprocal")
        oq = orc.quantize(to_np(x), tag, bits=2, group_size=32, div="reciprocal")
        np.testing.assert_array_equal(to_np(q.values), oq.values)
        np.testing.assert_array_equal(to_np(q.scale), oq.scale)


def test_large_seeded_pages_match_oracle():
    """Config-2 style pages (bf16, outlier channels) at a size the oracle finishes in seconds."""

    from dartkv_b200.synthetic import make_kvq

    keys, values, _ = make_kvq(1, 4, 8, 256, 128, dtype=torch.bfloat16)
    for bits in (2, 4, 8):
        q = dart.quantize(values.cuda(), bits=bits, group_size=64, metadata_dtype=torch.bfloat16)
        oq = orc.quantize(to_np(values), "bf16", bits=bits, group_size=64, md="bf16")
        np.testing.assert_array_equal(to_np(q.values), oq.values)
        np.testing.assert_array_equal(to_np(q.scale), oq.scale)
        np.testing.assert_array_equal(to_np(q.zero_point), oq.zero_point)
    m = dart.quantize_key_mixed(keys[:, :, :128].cuda(), group_size=128, promote_ratio=0.25)
    om = orc.quantize_key_mixed(to_np(keys[:, :, :128]), "bf16", group_size=128, ratio=0.25)
    np.testing.assert_array_equal(to_np(m.channel_indices), om.channel_indices)
    np.testing.assert_array_equal(to_np(m.low_values), om.low_values)
    np.testing.assert_array_equal(to_np(m.high_values), om.high_values)
    np.testing.assert_array_equal(to_np(m.scale), om.scale)
    np.testing.assert_array_equal(to_np(m.zero_point), om.zero_point)


def test_random_channel_selection_is_shared_across_the_batch():
    # src/dart/mixed.py:145-152: one random permutation per head, the same for every batch row
    keys = torch.randn(3, 2, 16, 32).cuda()
    mask, indices = dart.select_key_channels(keys, 0.25, strategy="random")
    assert tuple(mask.shape) == (3, 2, 32) and tuple(indices.shape) == (3, 2, 8)
    assert mask.dtype == torch.bool and int(mask.sum()) == 3 * 2 * 8
    assert torch.equal(indices[0], indices[1]) and torch.equal(indices[0], indices[2])
    for head in range(2):
        assert len(set(indices[0, head].tolist())) == 8
        assert torch.equal(mask[0, head].nonzero().flatten().cpu(), indices[0, head].sort().values.cpu())
    q = dart.quantize_key_mixed(keys, group_size=16, promote_ratio=0.25, strategy="random")
    assert tuple(q.high_values.shape[:3]) == (3, 2, 8) and torch.equal(q.channel_indices[0], q.channel_indices[2])
    assert (q.dequantize() - keys).abs().max() < 1.6
