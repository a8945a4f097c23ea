"""Parity of the CUDA path (through the C ABI) with the CPU oracle on identical seeded inputs.

Tolerances: out |gpu - ref| <= 2e-2 + 1e-2 |ref| for a bf16 cache, 5e-2 + 1e-2 |ref| for an fp8 cache,
every element, no mismatch budget; lse within 1e-3 (+1e-3 relative), infinities must match in sign.
Index handling is checked for integer equality."""
import math

import numpy as np
import pytest
import torch

from helpers import TOL_BF16, TOL_FP8, check_lse, check_out, csr_to_lists, load_golden, mxfp8_kv_to_rows, mxfp8_q_to_bf16
from opfoundry_b200 import api, synth

pytestmark = pytest.mark.gpu

SCALE = 1.0 / math.sqrt(192.0)


@pytest.fixture(scope="module", autouse=True)
def _need_gpu(built_lib):
    assert torch.cuda.is_available(), "these tests need a CUDA device"


def compare(case, oracle, tol, hint=None, subset=None):
    from gpu_util import run_gpu, run_oracle
    g_out, g_lse, plan = run_gpu(case, SCALE, valid_len_hint=hint)
    r_out, r_lse = run_oracle(oracle, case, SCALE, subset=subset)
    if subset is not None:
        g_out, g_lse, r_out, r_lse = g_out[subset], g_lse[subset], r_out[subset], r_lse[subset]
    e1 = check_out(g_out, r_out, **tol)
    e2 = check_lse(g_lse, r_lse)
    return e1, e2, plan


@pytest.mark.parametrize("topk", [1, 31, 32, 33, 63, 64, 65, 200])
def test_decode_bf16_tile_edges(oracle, topk):
    case = synth.make_decode_case(2, 128, 256, topk, seed=topk)
    compare(case, oracle, TOL_BF16)


@pytest.mark.parametrize("H", [16, 64, 128, 200])
def test_decode_bf16_heads(oracle, H):
    case = synth.make_decode_case(2, H, 512, 160, seed=H)
    compare(case, oracle, TOL_BF16)


def test_decode_bf16_config1(oracle):
    """BASELINE config 1: B=2, H=16, kv_len 4096 contiguous per sequence, top-k 2048."""
    case = synth.make_decode_case(2, 16, 4096, 2048, seed=2026)
    _, _, plan = compare(case, oracle, TOL_BF16)
    assert plan.info.num_partials > 0   # the list is split across CTA pairs and merged


def test_decode_bf16_padding_anywhere_and_poison(oracle):
    from gpu_util import poison_unselected
    case = synth.make_decode_case(3, 128, 1024, 300, pad_frac=0.3, scatter_pad=True, seed=5)
    case, n_poison = poison_unselected(case)
    assert n_poison > 0
    compare(case, oracle, TOL_BF16)


def test_decode_bf16_all_padding_query(oracle):
    case = synth.make_decode_case(3, 128, 256, 96, seed=6)
    case["indices"][1, :] = -1
    case["indices"][2, 5:] = -1
    from gpu_util import run_gpu
    g_out, g_lse, _ = run_gpu(case, SCALE)
    assert np.all(g_out[1] == 0) and np.all(np.isposinf(g_lse[1]))
    compare(case, oracle, TOL_BF16)


def test_decode_bf16_paged(oracle):
    case = synth.make_decode_case(4, 128, 1024, 257, paged=True, page_block_size=64, pad_frac=0.05, seed=8)
    compare(case, oracle, TOL_BF16)


def test_decode_bf16_mtp_two_rows_per_sequence(oracle):
    case = synth.make_decode_case(3, 128, 512, 128, s_q=2, paged=True, share_mtp="coin", seed=9)
    compare(case, oracle, TOL_BF16)


@pytest.mark.parametrize("topk", [1, 33, 64, 100])
def test_decode_fp8_tile_edges(oracle, topk):
    case = synth.make_decode_case(2, 128, 256, topk, fp8=True, seed=100 + topk)
    compare(case, oracle, TOL_FP8)


def test_decode_fp8_paged_padded_poison(oracle):
    from gpu_util import poison_unselected
    case = synth.make_decode_case(4, 128, 2048, 512, fp8=True, paged=True, pad_frac=0.05, seed=12)
    case, n_poison = poison_unselected(case)
    assert n_poison > 0
    _, _, plan = compare(case, oracle, TOL_FP8)


def test_decode_fp8_every_code_and_subnormals(oracle):
    """Cache bytes drawn from every finite e4m3 code, and a second cache made of subnormal codes only
    (|x| < 2^-6) with large scales so the result hangs on them: the in-kernel conversion must be exact."""
    rng = np.random.default_rng(77)
    base = synth.make_decode_case(2, 128, 256, 96, fp8=True, seed=78)
    for mode in ("all", "subnormal"):
        case = dict(base)
        kv = base["kv"].copy()
        n = kv.shape[0]
        if mode == "all":
            codes = rng.integers(0, 256, size=(n, 512)).astype(np.uint8)
            codes[(codes & 0x7F) == 0x7F] = 0x3A          # no NaN codes
            scales = rng.uniform(0.002, 0.02, size=(n, 4)).astype(np.float32)
        else:
            codes = (rng.integers(0, 8, size=(n, 512)) | (rng.integers(0, 2, size=(n, 512)) << 7)).astype(np.uint8)
            scales = np.full((n, 4), 256.0, np.float32)
        kv[:, :512] = codes
        kv[:, 512:528] = scales.view(np.uint8).reshape(n, 16)
        case["kv"] = kv
        compare(case, oracle, TOL_FP8)


def test_decode_fp8_small_heads(oracle):
    case = synth.make_decode_case(2, 16, 512, 130, fp8=True, paged=True, seed=13)
    compare(case, oracle, TOL_FP8)


def test_decode_fp8_golden_reference_vectors(oracle):
    """The reference's own fp8 case (golden vectors made by its CPU code) through the GPU path."""
    g = load_golden("ref_fp8_csr.npz")
    codec = load_golden("codec_e4m3.npz")
    B, H, sq = int(g["B"]), int(g["H"]), int(g["s_q"])
    q = mxfp8_q_to_bf16(g["q_nope"], g["q_scale"], g["q_rope"], codec["decode"].view(np.float32)).reshape(B * sq, H, 576)
    rows = mxfp8_kv_to_rows(g["kv_nope"], g["kv_scale"], g["kv_rope"])
    ind = csr_to_lists(g["kv_indptr"], g["kv_indices"], B, sq)
    case = dict(q=q, kv=rows, indices=ind, block_table=None, page_block_size=1, kv_batch_stride_rows=0, s_q=sq, fp8=True,
                H=H, topk=ind.shape[1])
    from gpu_util import run_gpu
    g_out, g_lse, _ = run_gpu(case, 1.0 / 24.0)
    check_out(g_out, g["out"], **TOL_FP8)
    check_lse(g_lse, g["lse"])


def test_decode_bf16_golden_reference_vectors(oracle):
    g = load_golden("ref_bf16_csr.npz")
    B, H, sq = int(g["B"]), int(g["H"]), int(g["s_q"])
    ind = csr_to_lists(g["kv_indptr"], g["kv_indices"], B, sq)
    case = dict(q=g["q"], kv=g["kv"], indices=ind, block_table=None, page_block_size=1, kv_batch_stride_rows=0, s_q=sq,
                fp8=False, H=H, topk=ind.shape[1])
    from gpu_util import run_gpu
    g_out, g_lse, _ = run_gpu(case, 1.0 / 24.0)
    check_out(g_out, g["out"], **TOL_BF16)
    check_lse(g_lse, g["lse"])


@pytest.mark.parametrize("fp8", [False, True])
def test_decode_padded_q_and_out_strides(oracle, fp8):
    """Q and out are views with padded head and row strides (the library takes element strides, as the
    reference's kargs do): the kernels read Q and write out through them."""
    from gpu_util import to_dev, run_oracle
    case = synth.make_decode_case(3, 128, 512, 150, fp8=fp8, paged=True, pad_frac=0.1, seed=61)
    d = to_dev(case)
    B, H = 3, 128
    q_big = torch.zeros(B, H + 3, 640, dtype=torch.bfloat16, device="cuda")
    q_big[:, :H, :576] = d["q"]
    q = q_big[:, :H, :576]
    out_big = torch.full((B, H + 1, 768), float("nan"), dtype=torch.bfloat16, device="cuda")
    out = out_big[:, :H, :512]
    lse = torch.empty(B, H, dtype=torch.float32, device="cuda")
    plan = api.mla_decode_plan_create(B, H, 150, 1)
    api.mla_decode_launch_pipeline(q, d["kv"], d["indices"], plan, SCALE, block_table=d["block_table"], page_block_size=64,
                                   out=out, lse=lse)
    torch.cuda.synchronize()
    r_out, r_lse = run_oracle(oracle, case, SCALE)
    g_out = out.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    check_out(g_out, r_out, **(TOL_FP8 if fp8 else TOL_BF16))
    check_lse(lse.cpu().numpy(), r_lse)
    assert torch.isnan(out_big[:, H:, :].float()).all() and torch.isnan(out_big[:, :, 512:].float()).all()   # nothing written outside


@pytest.mark.parametrize("fp8,page", [(False, 48), (True, 80), (True, 16)])
def test_decode_page_sizes(oracle, fp8, page):
    """Page sizes that are not powers of two take the divide / modulo translation; 16 the shift / mask one."""
    case = synth.make_decode_case(3, 128, 960, 200, fp8=fp8, paged=True, page_block_size=page, pad_frac=0.05, seed=70 + page)
    compare(case, oracle, TOL_FP8 if fp8 else TOL_BF16)


def test_prefill_bf16_small_causal(oracle):
    T, topk = 300, 128
    case = synth.make_prefill_case(T, 128, topk, seed=21)
    compare(case, oracle, TOL_BF16, hint=case["valid_len"])
    compare(case, oracle, TOL_BF16, hint=None)   # without the hint the -1 tail is masked, not skipped


def test_index_translation_is_bit_exact(oracle):
    case = synth.make_decode_case(5, 16, 4096, 700, paged=True, pad_frac=0.1, scatter_pad=True, s_q=1, seed=30)
    _, _, want = oracle.sparse_mla(case["q"], case["kv"], case["indices"], 1.0, block_table=case["block_table"],
                                   page_block_size=64, want_rows=True)
    got = api.debug_rows(torch.from_numpy(case["indices"]).cuda(), num_kv_rows=case["kv"].shape[0],
                         block_table=torch.from_numpy(case["block_table"]).cuda(), page_block_size=64)
    assert np.array_equal(got.cpu().numpy(), want)
    # contiguous cache, two query rows per sequence
    c2 = synth.make_decode_case(3, 16, 512, 64, s_q=2, seed=31)
    _, _, want = oracle.sparse_mla(c2["q"], c2["kv"], c2["indices"], 1.0, s_q=2, kv_batch_stride_rows=512, want_rows=True)
    got = api.debug_rows(torch.from_numpy(c2["indices"]).cuda(), s_q=2, num_kv_rows=c2["kv"].shape[0], kv_batch_stride_rows=512)
    assert np.array_equal(got.cpu().numpy(), want)
    # positions whose row falls outside the cache are masked, never dereferenced
    bad = torch.tensor([[5, 1 << 30, -7, 0]], dtype=torch.int32, device="cuda")
    got = api.debug_rows(bad, num_kv_rows=100)
    assert got.cpu().tolist() == [[5, -1, -1, 0]]


def test_pack_fp8_rows_bit_exact(oracle):
    rng = np.random.default_rng(40)
    latent = rng.standard_normal((1000, 512)).astype(np.float32)
    latent[7, :128] = 0
    latent[8, 3] = 1e6
    rope = synth.f32_to_bf16_bits(rng.standard_normal((1000, 64)).astype(np.float32))
    want = oracle.pack_fp8_rows(latent, rope)
    got = api.pack_fp8_rows(torch.from_numpy(latent).cuda(), torch.from_numpy(rope.view(np.int16)).cuda().view(torch.bfloat16))
    assert np.array_equal(got.cpu().numpy(), want)


def test_repeated_launches_are_deterministic(oracle):
    from gpu_util import run_gpu
    case = synth.make_decode_case(8, 128, 2048, 512, fp8=True, paged=True, seed=50)
    a_out, a_lse, _ = run_gpu(case, SCALE)
    b_out, b_lse, _ = run_gpu(case, SCALE)
    assert np.array_equal(a_out, b_out) and np.array_equal(a_lse, b_lse)


def test_bounded_wait_expires_and_reports(built_lib):
    """A device-side wait that nothing satisfies runs out after its budget, the kernel exits normally,
    the status word carries the code once, and the context keeps working."""
    import ctypes as C
    plan = api.mla_decode_plan_create(2, 16, 64, 1)
    result = torch.zeros(2, dtype=torch.int32, device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert built_lib.dsa_v32_selftest_wait_expiry(plan.workspace.data_ptr(), result.data_ptr(), 200, st) == 0
    a = api.AttnArgs()
    a.workspace = plan.workspace.data_ptr()
    assert built_lib.dsa_v32_device_status(C.byref(a), st) == 1001      # DSA_V32_ERR_DEVICE_WAIT, read and cleared
    assert result.cpu().tolist() == [1, 1]                              # the wait returned false and raised the abort flag
    assert built_lib.dsa_v32_device_status(C.byref(a), st) == 0
    assert built_lib.dsa_v32_selftest_wait_expiry(plan.workspace.data_ptr(), result.data_ptr(), 0, st) == -2
    # the context is intact: a normal launch on the same workspace still gives the right answer
    from gpu_util import run_gpu
    case = synth.make_decode_case(2, 16, 256, 64, fp8=False, seed=3)
    out, lse, _ = run_gpu(case, SCALE)
    assert np.all(np.isfinite(lse))


@pytest.mark.parametrize("fp8,H,s_q", [(True, 64, 2), (True, 16, 2), (False, 32, 4), (False, 64, 2)])
def test_mtp_shared_lists_stacked_rows(oracle, fp8, H, s_q):
    """Sequences whose MTP query rows share one index list run as one stacked item (rows gathered once);
    the result must equal the oracle's, which knows nothing of the stacking.  Small and large plans (with
    and without split items)."""
    from gpu_util import run_gpu, run_oracle
    for B, kv_len, topk in ((6, 1024, 512), (3, 4096, 2048)):
        case = synth.make_decode_case(B, H, kv_len, topk, s_q=s_q, fp8=fp8, paged=fp8, share_mtp="coin", seed=7 * H + s_q + B)
        if not case["mtp_shared"].any():
            case["mtp_shared"][0] = True
            case["indices"][1:s_q] = case["indices"][0]
        g_out, g_lse, plan = run_gpu(case, SCALE, mtp_shared=case["mtp_shared"])
        stacked = [w.stacked_rows for w in plan.read_works()[0]]
        assert max(stacked) == s_q
        r_out, r_lse = run_oracle(oracle, case, SCALE)
        check_out(g_out, r_out, **(TOL_FP8 if fp8 else TOL_BF16))
        check_lse(g_lse, r_lse)


@pytest.mark.parametrize("fp8", [True, False])
def test_host_buffer_pipeline_in_chunks(oracle, fp8):
    """The chunked host-buffer call (copies overlapped with the other chunks' kernels) against the oracle:
    pinned host inputs in, host outputs back, for a paged fp8 cache and a contiguous bf16 cache."""
    from gpu_util import to_dev, run_oracle
    B, H, topk = 8, 128, 256
    case = synth.make_decode_case(B, H, 1024, topk, fp8=fp8, paged=fp8, pad_frac=0.1, seed=77)
    d = to_dev(case)
    for chunks in (2, 4):
        plan = api.mla_decode_plan_create(B // chunks, H, topk, 1)
        out = torch.full((B, H, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
        lse = torch.full((B, H), float("nan"), dtype=torch.float32, device="cuda")
        q_dev, i_dev = torch.zeros_like(d["q"]), torch.zeros_like(d["indices"])
        a = api.make_args(q_dev, d["kv"], i_dev, plan, SCALE, out=out, lse=lse, block_table=d["block_table"],
                          page_block_size=case["page_block_size"], kv_batch_stride_rows=case["kv_batch_stride_rows"])
        q_host, i_host = d["q"].cpu().pin_memory(), d["indices"].cpu().pin_memory()
        out_host = torch.zeros(B, H, 512, dtype=torch.bfloat16).pin_memory()
        lse_host = torch.zeros(B, H, dtype=torch.float32).pin_memory()
        api.mla_decode_step_host(a, q_host, i_host, out_host, lse_host, num_chunks=chunks)
        torch.cuda.current_stream().synchronize()
        r_out, r_lse = run_oracle(oracle, case, SCALE)
        check_out(out_host.view(torch.int16).numpy().view(np.uint16), r_out, **(TOL_FP8 if fp8 else TOL_BF16))
        check_lse(lse_host.numpy(), r_lse)
        # the same with the kernels of two chunks side by side, each on half of the SMs
        sms = torch.cuda.get_device_properties(0).multi_processor_count // 4 * 2
        lanes = [api.mla_decode_plan_create(B // chunks, H, topk, 1, num_sms=sms) for _ in range(2)]
        out_host.zero_()
        lse_host.zero_()
        api.mla_decode_step_host(a, q_host, i_host, out_host, lse_host, num_chunks=chunks, lane_plans=lanes)
        torch.cuda.current_stream().synchronize()
        check_out(out_host.view(torch.int16).numpy().view(np.uint16), r_out, **(TOL_FP8 if fp8 else TOL_BF16))
        check_lse(lse_host.numpy(), r_lse)
