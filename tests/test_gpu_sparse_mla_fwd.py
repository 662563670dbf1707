"""Sparse MLA forward on the GPU against the reference fixtures and the fp32 oracle."""
import numpy as np
import pytest
import torch

from conftest import from_bits
from gpu_util import assert_close_fp, check_status
from oracle import dsa_oracle as orc

pytestmark = pytest.mark.gpu

IMPL_GENERIC, IMPL_TC = 1, 2


def _fwd(q, kv, idx, impl, q_start=None, **kw):
    import tilelang_ascend_b200 as dsa
    S, S_kv, D = q.shape[1], kv.shape[1], q.shape[-1]
    qs = S_kv - S if q_start is None else q_start
    out, lse = dsa.sparse_mla_fwd_raw(q.cuda(), kv.cuda(), idx.cuda(), sm_scale=D ** -0.5, q_start=qs, causal=True, dv=512,
                                      impl=impl, **kw)
    check_status()
    return out.cpu(), lse.cpu()


@pytest.mark.parametrize("impl", [IMPL_TC, IMPL_GENERIC])
@pytest.mark.parametrize("tag", ["a", "b"])
def test_reference_golden_fixture(golden, tag, impl):
    g = golden(f"sparse_mla_fwd_{tag}.npz")
    q, kv, idx = from_bits(g["q"]), from_bits(g["kv"]), torch.from_numpy(g["indices"])
    out, lse = _fwd(q, kv, idx, impl, q_start=int(g["q_start"]))
    assert_close_fp(out, from_bits(g["out"]), f"out vs reference golden ({tag})")  # the reference's own bar is rtol=atol=1e-2
    ref_o, ref_l = orc.sparse_mla_fwd(q, kv, idx, q_start_index_s=int(g["q_start"]))
    assert_close_fp(out, ref_o, "out vs oracle")
    assert_close_fp(lse, ref_l, "lse vs oracle")


@pytest.mark.parametrize("impl", [IMPL_TC, IMPL_GENERIC])
def test_cpu_runnable_config(impl):
    # B=1, S_q=128, S_kv=1024, H=16, topk=256, seed 0
    q, kv, idx = orc.make_sparse_mla_inputs(1, 128, 1024, 16, 256, seed=0)
    out, lse = _fwd(q, kv, idx, impl)
    ref_o, ref_l = orc.sparse_mla_fwd(q, kv, idx)
    assert_close_fp(out, ref_o, "out")
    assert_close_fp(lse, ref_l, "lse")


def test_reference_factory_signature_and_lse_keyword():
    import tilelang_ascend_b200 as dsa
    q, kv, idx = orc.make_sparse_mla_inputs(1, 16, 512, 128, 128, seed=2)
    kernel = dsa.sparse_attention_fwd(heads=128, dim=512, tail_dim=64, topk=128, kv_stride=1)
    out = kernel(q.cuda(), kv.cuda(), idx.cuda())
    assert isinstance(out, torch.Tensor) and out.dtype == torch.bfloat16 and tuple(out.shape) == (1, 16, 128, 512)
    out2, lse = dsa.sparse_attention_fwd(128, 512, 64, 128, 1, return_softmax_lse=True)(q.cuda(), kv.cuda(), idx.cuda())
    check_status()
    ref_o, ref_l = orc.sparse_mla_fwd(q, kv, idx)
    assert torch.equal(out, out2)
    assert_close_fp(out.cpu(), ref_o, "out")
    assert_close_fp(lse.cpu(), ref_l, "lse")
    assert dsa.sparse_attention_fwd(128, 512, 64, 128, 1) is kernel  # cached per argument tuple


def test_fp16_inputs():
    q, kv, idx = orc.make_sparse_mla_inputs(2, 8, 300, 128, 96, seed=3, dtype=torch.float16)
    for impl in (IMPL_TC, IMPL_GENERIC):
        out, lse = _fwd(q, kv, idx, impl)
        ref_o, ref_l = orc.sparse_mla_fwd(q, kv, idx)
        assert out.dtype == torch.float16
        assert_close_fp(out, ref_o, "out fp16")
        assert_close_fp(lse, ref_l, "lse fp16")


@pytest.mark.parametrize("impl", [IMPL_TC, IMPL_GENERIC])
def test_padding_sentinels_masked_and_empty_rows(impl):
    B, S, S_kv, H, topk = 2, 6, 200, 32, 64
    q, kv, idx = orc.make_sparse_mla_inputs(B, S, S_kv, H, topk, seed=4)
    idx[0, 0, 0, :] = -1                       # a query with no key at all
    idx[0, 1, 0, ::2] = S_kv                   # the torch golden's sentinel
    idx[0, 2, 0, 5:] = -1                      # -1 terminated list
    idx[1, 0, 0, :32] = -1                     # a whole first tile empty, keys only later
    idx[1, 1, 0, 3] = S_kv - 1                 # beyond the causal limit of query 1
    idx[1, 2, 0, 7] = 10 ** 6                  # out of range
    out, lse = _fwd(q, kv, idx, impl)
    ref_o, ref_l = orc.sparse_mla_fwd(q, kv, idx)
    assert_close_fp(out, ref_o, "out")
    assert_close_fp(lse, ref_l, "lse")
    assert torch.all(out[0, 0] == 0) and torch.all(torch.isinf(lse[0, 0]))


def test_ragged_topk_and_head_counts():
    for H, topk in ((1, 40), (17, 8), (64, 72), (128, 200), (130, 33)):
        q, kv, idx = orc.make_sparse_mla_inputs(1, 5, 400, H, topk, seed=H)
        ref_o, ref_l = orc.sparse_mla_fwd(q, kv, idx)
        for impl in (IMPL_TC, IMPL_GENERIC):
            out, lse = _fwd(q, kv, idx, impl)
            assert_close_fp(out, ref_o, f"out H={H} topk={topk}")
            assert_close_fp(lse, ref_l, f"lse H={H} topk={topk}")


def test_large_scores_need_rescaling():
    # a growing maximum across tiles exercises the accumulator rescale path
    q, kv, idx = orc.make_sparse_mla_inputs(1, 4, 600, 128, 512, seed=6)
    kv = (kv.float() * torch.linspace(0.2, 3.0, 600).view(1, -1, 1, 1)).to(torch.bfloat16)
    idx = torch.sort(idx, dim=-1).values  # ascending positions -> growing score magnitude
    out, lse = _fwd(q, kv, idx, IMPL_TC)
    ref_o, ref_l = orc.sparse_mla_fwd(q, kv, idx)
    assert_close_fp(out, ref_o, "out")
    assert_close_fp(lse, ref_l, "lse")


def test_decode_shape_small():
    # decode: one query per sequence, non-causal sampling over the whole cache
    B, S_kv, H, topk = 4, 4096, 128, 512
    q, kv, idx = orc.make_sparse_mla_inputs(B, 1, S_kv, H, topk, seed=7, causal=False)
    out, lse = _fwd(q, kv, idx, IMPL_TC)
    ref_o, ref_l = orc.sparse_mla_fwd(q, kv, idx)
    assert_close_fp(out, ref_o, "out")
    assert_close_fp(lse, ref_l, "lse")


def test_paged_front_end_matches_numpy_golden(golden):
    import tilelang_ascend_b200 as dsa
    g = golden("sfa_numpy_golden.npz")
    q, kv = from_bits(g["q"]), from_bits(g["kv"])
    idx = torch.from_numpy(g["indices"])
    act_q, act_kv = torch.from_numpy(g["act_q"]), torch.from_numpy(g["act_kv"])
    # BSND
    out = dsa.sparse_attn_tilelang(q[..., :512].cuda(), kv[..., :512].cuda(), None, idx.cuda(), 576 ** -0.5, 1, act_q, act_kv,
                                   query_rope=q[..., 512:].cuda(), key_rope=kv[..., 512:].cuda())
    check_status()
    for b in range(q.shape[0]):
        aq = int(act_q[b])
        assert_close_fp(out[b, :aq].cpu(), torch.from_numpy(g["out"][b, :aq]), "BSND vs NumPy golden")
    # paged: scatter the same keys into shuffled 16-token blocks
    bs, B, S_kv = 16, kv.shape[0], kv.shape[1]
    nblk = S_kv // bs
    perm = torch.randperm(B * nblk, generator=torch.Generator().manual_seed(0))
    table = perm.view(B, nblk).to(torch.int32)
    paged = torch.zeros((B * nblk, bs, 1, 576), dtype=kv.dtype)
    for b in range(B):
        for j in range(nblk):
            paged[table[b, j]] = kv[b, j * bs:(j + 1) * bs]
    out_p = dsa.sparse_attn_tilelang(q[..., :512].cuda(), paged[..., :512].cuda(), None, idx.cuda(), 576 ** -0.5, 1, act_q, act_kv,
                                     query_rope=q[..., 512:].cuda(), key_rope=paged[..., 512:].cuda(), layout_kv="PA_BSND",
                                     block_table=table.cuda())
    check_status()
    for b in range(B):
        aq = int(act_q[b])
        assert torch.equal(out_p[b, :aq], out[b, :aq])


def test_rejects_bad_inputs():
    import tilelang_ascend_b200 as dsa
    q, kv, idx = orc.make_sparse_mla_inputs(1, 4, 64, 16, 64, seed=0)
    k = dsa.sparse_attention_fwd(16, 512, 64, 64, 1)
    with pytest.raises(ValueError):
        k(q.cuda().transpose(1, 2), kv.cuda(), idx.cuda())          # not contiguous
    with pytest.raises(ValueError):
        k(q.cuda().half(), kv.cuda(), idx.cuda())                    # dtype
    with pytest.raises(ValueError):
        k(q.cuda(), kv, idx.cuda())                                  # device
    with pytest.raises(ValueError):
        k(q.cuda(), kv.cuda(), idx.cuda().long())                    # index dtype
    with pytest.raises(AssertionError):
        dsa.sparse_attention_fwd(16, 512, 64, 100, 1)                # topk % block_I
    with pytest.raises(AssertionError):
        dsa.sparse_attention_fwd(16, 512, 64, 64, 1, is_causal=False)


def test_host_buffer_pipeline_matches_direct_call():
    import tilelang_ascend_b200 as dsa
    B, S, S_kv, H, topk = 1, 100, 512, 128, 128
    q, kv, idx = orc.make_sparse_mla_inputs(B, S, S_kv, H, topk, seed=8)
    kernel = dsa.sparse_attention_fwd(H, 512, 64, topk, 1, return_softmax_lse=True)
    ref_o, ref_l = kernel(q.cuda(), kv.cuda(), idx.cuda())
    pipe = dsa.HostPipelinedForward(kernel, q.shape, kv.shape, idx.shape, 512, chunks=7)
    out_h = torch.empty((B, S, H, 512), dtype=torch.bfloat16).pin_memory()
    lse_h = torch.empty((B, S, H), dtype=torch.float32).pin_memory()
    for _ in range(2):  # staging buffers are reused across calls
        out_h.zero_()
        pipe(q.pin_memory(), kv.pin_memory(), idx.pin_memory(), out_h, lse_h)
        torch.cuda.synchronize()
        check_status()
        assert torch.equal(out_h, ref_o.cpu()) and torch.equal(lse_h, ref_l.cpu())
    with pytest.raises(ValueError):
        pipe(q, kv.pin_memory(), idx.pin_memory(), out_h, lse_h)  # not pinned


@pytest.mark.parametrize("nsplit", [2, 3, 5, 16])
def test_split_kv_matches_unsplit_and_oracle(nsplit):
    """Keys of a query split over several work units + combine: same result as one unit per query.  topk 320 = 5 tiles
    of 64, so 2 and 3 give uneven shares, 5 one tile each, 16 leaves most shares without a tile; a short query (fewer
    keys than tiles) and -1 padding are in the mix through the causal sampling of the first rows."""
    q, kv, idx = orc.make_sparse_mla_inputs(2, 6, 400, 128, 320, seed=9)
    idx[0, 0, 0, 40:] = -1  # one query with a single partly filled tile
    one_o, one_l = _fwd(q, kv, idx, IMPL_TC, nsplit=1)
    spl_o, spl_l = _fwd(q, kv, idx, IMPL_TC, nsplit=nsplit)
    assert_close_fp(spl_o, one_o, "split vs unsplit out")
    assert_close_fp(spl_l, one_l, "split vs unsplit lse")
    ref_o, ref_l = orc.sparse_mla_fwd(q, kv, idx)
    assert_close_fp(spl_o, ref_o, "out vs oracle")
    assert_close_fp(spl_l, ref_l, "lse vs oracle")


def test_pair_kernel_agrees_with_split_kernel_and_repeats_bit_identically(monkeypatch):
    """The default kernel (cta_group::2 MMAs, heads split over the SM pair) against the kernel it replaced (each CTA all
    heads and half of the dims), on items of several tiles with causal (short) rows among them; and two launches of the
    default kernel give the same bits: every accumulator has one issuing thread, so the summation order is fixed."""
    q, kv, idx = orc.make_sparse_mla_inputs(1, 96, 2048, 128, 512, seed=21)
    monkeypatch.delenv("DSA_FWD_KERNEL", raising=False)
    a_o, a_l = _fwd(q, kv, idx, IMPL_TC)
    b_o, b_l = _fwd(q, kv, idx, IMPL_TC)
    assert torch.equal(a_o, b_o) and torch.equal(a_l, b_l)
    monkeypatch.setenv("DSA_FWD_KERNEL", "split")
    s_o, s_l = _fwd(q, kv, idx, IMPL_TC)
    assert_close_fp(a_o, s_o, "pair vs split kernel out")
    assert_close_fp(a_l, s_l, "pair vs split kernel lse")
    ref_o, ref_l = orc.sparse_mla_fwd(q, kv, idx)
    assert_close_fp(a_o, ref_o, "out vs oracle")
    assert_close_fp(a_l, ref_l, "lse vs oracle")


def test_units_of_one_tile_between_empty_units_repeat_bit_identically():
    """Many work units of a single tile with empty units between them (5 tiles over 16 shares): the two Q K^T issuing
    threads alternate, each skipping every other unit, which is where a hand-over that lets a thread run a unit ahead would
    show as a result that changes between launches."""
    q, kv, idx = orc.make_sparse_mla_inputs(2, 40, 400, 128, 320, seed=13)
    first_o, first_l = _fwd(q, kv, idx, IMPL_TC, nsplit=16)
    ref_o, ref_l = orc.sparse_mla_fwd(q, kv, idx)
    assert_close_fp(first_o, ref_o, "out vs oracle")
    assert_close_fp(first_l, ref_l, "lse vs oracle")
    for _ in range(10):
        o, l = _fwd(q, kv, idx, IMPL_TC, nsplit=16)
        assert torch.equal(o, first_o) and torch.equal(l, first_l)


def test_split_kv_is_chosen_for_a_few_sequences_and_handles_absent_queries():
    """Decode of 4 sequences: the library splits on its own (fewer queries than SM pairs); per-sequence lengths, one
    sequence without its query (q_len 0): out = 0 and lse = -inf there."""
    import tilelang_ascend_b200 as dsa
    from tilelang_ascend_b200 import _lib
    B, S_kv, H, topk = 4, 2048, 128, 512
    g = torch.Generator().manual_seed(4)
    q = torch.randn((B, 1, H, 576), generator=g).to(torch.bfloat16)
    kv = torch.randn((B, S_kv, 1, 576), generator=g).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(S_kv, generator=g)[:topk] for _ in range(B)]).to(torch.int32).view(B, 1, 1, topk)
    assert int(_lib.load().dsa_sparse_mla_fwd_splitkv_nsplit(B, 1, H, topk)) > 1
    q_len = torch.tensor([1, 1, 0, 1], dtype=torch.int32)
    kv_len = torch.tensor([S_kv, 1500, S_kv, S_kv], dtype=torch.int32)
    out, lse = dsa.sparse_mla_fwd_raw(q.cuda(), kv.cuda(), idx.cuda(), sm_scale=576 ** -0.5, q_start=0, causal=False, dv=512,
                                      q_len_b=q_len.cuda(), kv_len_b=kv_len.cuda())
    check_status()
    one, one_l = dsa.sparse_mla_fwd_raw(q.cuda(), kv.cuda(), idx.cuda(), sm_scale=576 ** -0.5, q_start=0, causal=False, dv=512,
                                        q_len_b=q_len.cuda(), kv_len_b=kv_len.cuda(), nsplit=1)
    check_status()
    assert_close_fp(out.cpu(), one.cpu(), "auto split vs unsplit out")
    assert_close_fp(lse.cpu(), one_l.cpu(), "auto split vs unsplit lse")
    gen, gen_l = dsa.sparse_mla_fwd_raw(q.cuda(), kv.cuda(), idx.cuda(), sm_scale=576 ** -0.5, q_start=0, causal=False, dv=512,
                                        q_len_b=q_len.cuda(), kv_len_b=kv_len.cuda(), impl=_lib.IMPL_GENERIC)
    check_status()
    assert_close_fp(gen.cpu(), one.cpu(), "CUDA-core kernel vs tensor-core kernel out")
    # the absent query's row is written by every kernel (the NumPy golden leaves it zero): out = 0, lse = -inf
    for o, l in ((out, lse), (one, one_l), (gen, gen_l)):
        assert torch.count_nonzero(o[2]).item() == 0 and torch.isinf(l[2]).all() and (l[2] < 0).all()


def test_split_kv_fp16_paged():
    """Split-KV through a block table and in float16: same answer as one unit per query on the same paged cache."""
    import tilelang_ascend_b200 as dsa
    B, S_kv, H, topk, bs = 3, 1024, 128, 256, 64
    g = torch.Generator().manual_seed(12)
    q = torch.randn((B, 1, H, 576), generator=g).to(torch.float16)
    kv = torch.randn((B, S_kv, 1, 576), generator=g).to(torch.float16)
    idx = torch.stack([torch.randperm(S_kv, generator=g)[:topk] for _ in range(B)]).to(torch.int32).view(B, 1, 1, topk)
    nblk = S_kv // bs
    table = torch.randperm(B * nblk, generator=g).view(B, nblk).to(torch.int32)
    paged = torch.zeros((B * nblk, bs, 1, 576), dtype=kv.dtype)
    for b in range(B):
        for j in range(nblk):
            paged[table[b, j]] = kv[b, j * bs:(j + 1) * bs]
    kw = dict(sm_scale=576 ** -0.5, q_start=0, causal=False, dv=512, block_table=table.cuda(), block_size=bs)
    one, one_l = dsa.sparse_mla_fwd_raw(q.cuda(), paged.cuda(), idx.cuda(), nsplit=1, **kw)
    spl, spl_l = dsa.sparse_mla_fwd_raw(q.cuda(), paged.cuda(), idx.cuda(), nsplit=2, **kw)
    check_status()
    assert_close_fp(spl.cpu(), one.cpu(), "paged fp16 split vs unsplit out")
    assert_close_fp(spl_l.cpu(), one_l.cpu(), "paged fp16 split vs unsplit lse")
    ref_o, ref_l = orc.sparse_mla_fwd(q, kv, idx, q_start_index_s=10 ** 9)
    assert_close_fp(spl.cpu(), ref_o, "out vs oracle")
    assert_close_fp(spl_l.cpu(), ref_l, "lse vs oracle")


def test_tensor_core_forward_without_rope_dims():
    """D = DV = 512 (keys are the values, no rope dims): tensor-core kernel against the oracle and the CUDA-core kernel."""
    import tilelang_ascend_b200 as dsa
    from tilelang_ascend_b200 import _lib
    B, S, S_kv, H, topk = 2, 5, 400, 64, 192
    q, kv, idx = orc.make_sparse_mla_inputs(B, S, S_kv, H, topk, D=512, seed=12)
    scale = 512 ** -0.5
    qc, kvc, ic = q.cuda(), kv.cuda(), idx.cuda()
    out, lse = dsa.sparse_mla_fwd_raw(qc, kvc, ic, sm_scale=scale, q_start=S_kv - S, causal=True, dv=512, impl=_lib.IMPL_TENSOR_CORE)
    out_g, lse_g = dsa.sparse_mla_fwd_raw(qc, kvc, ic, sm_scale=scale, q_start=S_kv - S, causal=True, dv=512, impl=_lib.IMPL_GENERIC)
    check_status()
    ref_o, ref_l = orc.sparse_mla_fwd(q, kv, idx, sm_scale=scale, dv=512)
    assert_close_fp(out.cpu(), ref_o, "out (D=512, tensor core)")
    assert_close_fp(lse.cpu(), ref_l, "lse (D=512, tensor core)")
    assert_close_fp(out.cpu(), out_g.cpu(), "tensor core vs CUDA core")
    assert_close_fp(lse.cpu(), lse_g.cpu(), "lse tensor core vs CUDA core")


def test_bounded_wait_gives_up_and_reports_status():
    """The path every in-kernel wait takes when its hand-over never comes, exercised without a fault or a hang: a self-test
    kernel waits about a millisecond on a barrier that nothing completes, gives up, sets the status word and returns.  While
    the word is set a forward launch returns at once; reading the status clears it and the next launch computes again."""
    import tilelang_ascend_b200 as dsa
    from tilelang_ascend_b200 import _lib
    check_status()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.check(_lib.load().dsa_selftest_bounded_wait(2_000_000, flag.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert int(flag.item()) == 1
    q, kv, idx = orc.make_sparse_mla_inputs(1, 4, 256, 128, 64, seed=2)
    out = torch.full((1, 4, 128, 512), 7.0, dtype=torch.bfloat16, device="cuda")
    dsa.sparse_mla_fwd_raw(q.cuda(), kv.cuda(), idx.cuda(), sm_scale=576 ** -0.5, q_start=252, causal=True, dv=512, out=out)
    assert dsa.kernel_status() == 1            # reported once ...
    assert bool((out == 7.0).all())            # ... and the launch made while it was set wrote nothing
    assert dsa.kernel_status() == 0            # ... then cleared
    got, lse = dsa.sparse_mla_fwd_raw(q.cuda(), kv.cuda(), idx.cuda(), sm_scale=576 ** -0.5, q_start=252, causal=True, dv=512, out=out)
    check_status()
    ref_o, ref_l = orc.sparse_mla_fwd(q, kv, idx)
    assert_close_fp(got.cpu(), ref_o, "out after the status was cleared")


def test_debug_check_flags_repeated_indices(monkeypatch):
    import tilelang_ascend_b200 as dsa
    q, kv, idx = orc.make_sparse_mla_inputs(1, 4, 256, 16, 64, seed=3)
    monkeypatch.setenv("DSA_DEBUG_BOUNDS", "1")
    dsa.sparse_mla_fwd_raw(q.cuda(), kv.cuda(), idx.cuda(), sm_scale=576 ** -0.5, q_start=252, causal=True, dv=512)
    idx[0, 2, 0, 5] = idx[0, 2, 0, 9]
    with pytest.raises(ValueError, match="more than once"):
        dsa.sparse_mla_fwd_raw(q.cuda(), kv.cuda(), idx.cuda(), sm_scale=576 ** -0.5, q_start=252, causal=True, dv=512)
    check_status()


@pytest.mark.parametrize("S,m,n,H", [(200, 30, 2, 128), (160, 12, 4, 128), (75, 1, 3, 128), (90, 89, 2, 128), (60, 7, 3, 256), (50, 20, 2, 72)])
def test_split_tail_rows_are_combined_and_all_other_rows_stay_bit_equal(S, m, n, H):
    """Only the first m queries of a launch split into n shares (the tail that a persistent kernel reaches last): those rows
    agree with the unsplit call and the oracle within the usual tolerance, every other row is bit-equal to the unsplit call."""
    import tilelang_ascend_b200 as dsa
    q, kv, idx = orc.make_sparse_mla_inputs(1, S, 600, H, 320, seed=S + m)
    whole_o, whole_l = _fwd(q, kv, idx, IMPL_TC, nsplit=1)
    out, lse = dsa.sparse_mla_fwd_raw(q.cuda(), kv.cuda(), idx.cuda(), sm_scale=576 ** -0.5, q_start=600 - S, causal=True, dv=512,
                                      nsplit=n, split_queries=m)
    check_status()
    out, lse = out.cpu(), lse.cpu()
    assert torch.equal(out[:, m:], whole_o[:, m:]) and torch.equal(lse[:, m:], whole_l[:, m:])
    assert_close_fp(out[:, :m], whole_o[:, :m], "split rows vs unsplit out")
    assert_close_fp(lse[:, :m], whole_l[:, :m], "split rows vs unsplit lse")
    ref_o, ref_l = orc.sparse_mla_fwd(q, kv, idx)
    assert_close_fp(out, ref_o, "out vs oracle")
    assert_close_fp(lse, ref_l, "lse vs oracle")
    kernel = dsa.sparse_attention_fwd(H, 512, 64, 320, 1, return_softmax_lse=True)
    k_o, k_l = kernel(q.cuda(), kv.cuda(), idx.cuda(), split_tail=(m, n))
    assert torch.equal(k_o.cpu(), out) and torch.equal(k_l.cpu(), lse)
