"""Host-side generators: e4m3 packing equals the oracle's codec bit for bit; index lists are unique,
in range, causal where promised, and padded with -1 where promised."""
import numpy as np

from opfoundry_b200 import synth


def test_numpy_e4m3_encoder_matches_oracle(oracle):
    rng = np.random.default_rng(1)
    xs = np.concatenate([
        rng.standard_normal(30000) * 300, rng.standard_normal(30000) * 0.01,
        np.array([0.0, -0.0, 448.0, 449.9, 1e30, -1e30, np.inf, -np.inf, np.nan, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -10,
                  2.0 ** -11, 3 * 2.0 ** -10])]).astype(np.float32)
    want = np.array([oracle.lib().dsa_oracle_f32_to_e4m3(float(x)) for x in xs], np.uint8)
    got = synth.f32_to_e4m3_bits(xs)
    assert np.array_equal(want, got)


def test_pack_fp8_rows_matches_oracle(oracle):
    rng = np.random.default_rng(2)
    latent = rng.standard_normal((37, 512)).astype(np.float32)
    latent[3, 128:256] = 0.0  # an all-zero group keeps scale 1.0
    rope = synth.f32_to_bf16_bits(rng.standard_normal((37, 64)).astype(np.float32))
    assert np.array_equal(synth.pack_fp8_rows(latent, rope), oracle.pack_fp8_rows(latent, rope))
    deq = oracle.dequant_fp8_rows(oracle.pack_fp8_rows(latent, rope))
    assert np.max(np.abs(deq[:, :512] - latent)) < 0.3  # e4m3 keeps 3 mantissa bits


def test_bf16_round_trip():
    x = np.random.default_rng(0).standard_normal(1000).astype(np.float32)
    b = synth.f32_to_bf16_bits(x)
    assert np.max(np.abs(synth.bf16_bits_to_f32(b) - x) / np.abs(x)) < 2 ** -8


def test_decode_case_invariants():
    c = synth.make_decode_case(3, 4, 256, 64, s_q=2, fp8=True, paged=True, pad_frac=0.25, share_mtp="coin", seed=7)
    assert c["q"].shape == (6, 4, 576) and c["kv"].shape == (3 * 256, 656)
    bt = c["block_table"]
    assert sorted(bt.reshape(-1).tolist()) == list(range(3 * 4))
    for r in range(6):
        row = c["indices"][r]
        assert np.all(row[48:] == -1) and np.all(row[:48] >= 0) and np.all(row[:48] < 256)
        assert len(set(row[:48].tolist())) == 48
    c2 = synth.make_decode_case(3, 4, 256, 64, s_q=2, fp8=True, paged=True, pad_frac=0.25, share_mtp="coin", seed=7)
    assert np.array_equal(c["kv"], c2["kv"]) and np.array_equal(c["indices"], c2["indices"])
    c3 = synth.make_decode_case(2, 2, 128, 32, pad_frac=0.25, scatter_pad=True, seed=1)
    assert np.all((c3["indices"] == -1).sum(axis=1) == 8)
    assert not np.all(c3["indices"][:, 24:] == -1)


def test_prefill_case_invariants():
    c = synth.make_prefill_case(40, 2, 16, seed=3)
    for t in range(40):
        row = c["indices"][t]
        n = min(t + 1, 16)
        assert np.all(row[:n] >= 0) and np.all(row[:n] <= t) and np.all(row[n:] == -1)
        assert len(set(row[:n].tolist())) == n
    assert np.array_equal(c["valid_len"], np.minimum(np.arange(40) + 1, 16))
