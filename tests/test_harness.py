"""The verify-then-bench harness: flag parsing (CPU) and a verify run per mode (GPU)."""
import pytest

import mla_decode_harness as H


def test_flags_parse_like_the_reference_cli():
    o = H.parse_args(["-dtype", "bf16", "-h_q=16", "-b", "2", "-s=4096", "-s_q", "2", "--varlen", "--verify"])
    assert (o["dtype"], o["h_q"], o["b"], o["s"], o["s_q"], o["varlen"], o["verify"]) == ("bf16", 16, 2, 4096, 2, True, True)
    d = H.parse_args([])
    assert (d["dtype"], d["h_q"], d["b"], d["s"], d["s_q"], d["varlen"], d["verify"]) == ("fp8", 128, 128, 1024, 1, False, False)
    o = H.parse_args(["-mode=prefill", "-dtype", "bf16", "-topk", "512", "-pad_frac", "0.25", "-warmup=3", "-iters", "5"])
    assert (o["mode"], o["topk"], o["pad_frac"], o["warmup"], o["iters"]) == ("prefill", 512, 0.25, 3, 5)
    for bad in (["-bogus", "1"], ["-b", "0"], ["-dtype", "fp4"], ["--what"], ["-mode", "prefill"], ["-b"]):
        with pytest.raises(ValueError):
            H.parse_args(bad)


def test_varlen_lengths_follow_the_reference_range():
    o = H.parse_args(["-b", "64", "-s", "300", "--varlen"])
    lens = H.sequence_lengths(o)
    assert lens.shape == (64,) and lens.min() >= 5 and lens.max() <= 300 and len(set(lens.tolist())) > 8
    assert (H.sequence_lengths(H.parse_args(["-b", "4", "-s", "3", "--varlen"])) == 3).all()
    assert (H.sequence_lengths(H.parse_args(["-b", "4", "-s", "77"])) == 77).all()


@pytest.mark.gpu
@pytest.mark.parametrize("argv", [
    ["-dtype", "bf16", "-h_q", "16", "-b", "2", "-s", "4096", "--verify"],                       # configuration 1
    ["-dtype", "fp8", "-h_q", "128", "-b", "6", "-s", "3000", "-s_q", "2", "--varlen", "--verify"],
    ["-dtype", "bf16", "-mode", "prefill", "-s", "600", "-topk", "256", "--verify"],
])
def test_verify_then_bench(built_lib, oracle, argv, capsys):
    assert H.main(argv + ["-warmup", "3", "-iters", "5"]) == 0
    text = capsys.readouterr().out
    assert "Validation passed" in text and "LSE validation passed" in text and "MLA decode performance" in text
