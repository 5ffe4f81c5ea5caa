"""Element conversions of the oracle: FP8 E4M3FN, BF16 and F16.

The reference delegates BF16/F16 rounding to the crate `half` 2.7.1
(Cargo.lock) and encodes FP8 with a nearest-candidate scan
(crates/loom-kernels/src/quantization.rs:32-56). The oracle restates both;
these tests cross-check them against torch's casts and against a direct
bit-level encoder on every code boundary and a dense sample.
"""

import numpy as np
import torch

from oracle import binding as ob


def _interesting_f32(rng, count):
    bits = rng.integers(0, 2**32, size=count, dtype=np.uint64).astype(np.uint32)
    values = bits.view(np.float32)
    return values[np.isfinite(values)]


def test_fp8_decode_table_matches_torch():
    codes = np.arange(256, dtype=np.uint8)
    ours = ob.fp8_to_f32(codes)
    theirs = torch.from_numpy(codes).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    finite = np.isfinite(theirs)
    assert np.array_equal(np.isnan(ours), np.isnan(theirs))
    assert np.array_equal(ours[finite], theirs[finite])
    assert np.array_equal(np.signbit(ours), np.signbit(theirs))


def test_fp8_scan_equals_direct_encoder_on_boundaries_and_samples():
    rng = np.random.default_rng(11)
    decoded = ob.fp8_to_f32(np.arange(0x7F, dtype=np.uint8)).astype(np.float64)
    midpoints = ((decoded[:-1] + decoded[1:]) / 2).astype(np.float32)
    around = []
    for centre in np.concatenate([decoded.astype(np.float32), midpoints, np.float32([448, 464, 1e-30])]):
        c = np.float32(centre)
        around += [c, np.nextafter(c, np.float32(np.inf)), np.nextafter(c, np.float32(-np.inf))]
    dense = np.concatenate([
        np.float32(around),
        -np.float32(around),
        (rng.standard_normal(200_000) * 3).astype(np.float32),
        (rng.standard_normal(50_000) * 200).astype(np.float32),
        (rng.standard_normal(50_000) * 0.01).astype(np.float32),
        _interesting_f32(rng, 100_000),
        np.float32([0.0, -0.0, np.inf, -np.inf]),
    ])
    scan = ob.fp8_from_f32(dense)
    lib = ob.lib()
    direct = np.array([lib.oracle_fp8_e4m3fn_from_f32_direct(float(v)) for v in dense[:60_000]], dtype=np.uint8)
    assert np.array_equal(scan[:60_000], direct)
    # torch's cast is round-to-nearest-even without saturation; compare where
    # the input is inside the finite range.
    inside = np.abs(dense) < 448
    theirs = torch.from_numpy(dense[inside]).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(scan[inside], theirs)
    assert ob.fp8_from_f32([448.0, 1e9, np.inf, -500.0]).tolist() == [0x7E, 0x7E, 0x7E, 0xFE]
    assert ob.fp8_from_f32([np.nan])[0] & 0x7F == 0x7F
    assert ob.fp8_from_f32([-0.0])[0] == 0x80


def test_bf16_and_f16_round_like_torch():
    rng = np.random.default_rng(12)
    values = np.concatenate([
        (rng.standard_normal(200_000) * 2).astype(np.float32),
        _interesting_f32(rng, 200_000),
        np.float32([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 2.99e-8, 6.1e-5]),
    ])
    # exact ties: a BF16 value plus half a BF16 ulp
    base = (rng.integers(0, 2**16, size=20_000).astype(np.uint32) << 16)
    ties = (base | 0x8000).view(np.float32)
    ties = ties[np.isfinite(ties)]
    values = np.concatenate([values, ties])
    t = torch.from_numpy(values)
    assert np.array_equal(ob.f32_to_bf16(values), t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16))
    assert np.array_equal(ob.f32_to_f16(values), t.to(torch.float16).view(torch.int16).numpy().view(np.uint16))


def test_widening_is_exact():
    codes = np.arange(2**16, dtype=np.uint16)
    t = torch.from_numpy(codes.view(np.int16))
    bf = t.view(torch.bfloat16).to(torch.float32).numpy()
    hf = t.view(torch.float16).to(torch.float32).numpy()
    ours_bf, ours_hf = ob.bf16_to_f32(codes), ob.f16_to_f32(codes)
    assert np.array_equal(ours_bf.view(np.uint32)[~np.isnan(bf)], bf.view(np.uint32)[~np.isnan(bf)])
    assert np.array_equal(ours_hf.view(np.uint32)[~np.isnan(hf)], hf.view(np.uint32)[~np.isnan(hf)])
    assert np.array_equal(np.isnan(ours_hf), np.isnan(hf))
