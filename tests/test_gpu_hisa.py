"""HISA block-sparse indexer logits on the GPU against the oracle."""
import pytest
import torch

from gpu_util import check_status
from oracle import dsa_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("S,S_kv,H,D,bs,topk,dtype,wdtype", [
    (64, 4096, 32, 128, 128, 8, torch.float16, torch.float16),     # the reference test's shape family (fp16): tensor-core kernel
    (40, 5000, 64, 128, 128, 12, torch.bfloat16, torch.float32),   # tensor-core kernel, S_kv not a multiple of the block, 64 heads
    (9, 700, 20, 128, 128, 4, torch.bfloat16, torch.bfloat16),     # tensor-core kernel, head count below 64 and not a multiple of 16
    (11, 900, 40, 128, 128, 4, torch.bfloat16, torch.float32),     # 40 heads: UMMA N = 48, accumulator columns 48..63 are never written
    (33, 1000, 64, 128, 64, 12, torch.bfloat16, torch.float32),    # S_kv not a multiple of the block: the last block is cut
    (5, 300, 7, 64, 48, 4, torch.bfloat16, torch.bfloat16),        # block size that is not a multiple of 32, odd head count
])
@pytest.mark.parametrize("loader", ["tma", "cp_async"])
def test_block_sparse_logits_match_oracle(S, S_kv, H, D, bs, topk, dtype, wdtype, loader, monkeypatch):
    import tilelang_ascend_b200 as dsa
    # the tensor-core kernel fetches a block with two TMA tile loads; DSA_HISA_NO_TMA=1 selects its cp.async loaders
    monkeypatch.setenv("DSA_HISA_NO_TMA", "1" if loader == "cp_async" else "0")
    g = torch.Generator().manual_seed(S)
    q = (torch.rand((S, H, D), generator=g) - 0.5).to(dtype)
    k = (torch.rand((S_kv, D), generator=g) - 0.5).to(dtype)
    w = (torch.rand((S, H), generator=g) - 0.3).to(wdtype)
    ks = torch.randint(0, S_kv // 8, (S,), generator=g, dtype=torch.int32)
    ke = (torch.arange(1, S + 1, dtype=torch.int32) * (S_kv // S)).clamp(max=S_kv)
    blk = torch.randint(0, (S_kv + bs - 1) // bs, (S, topk), generator=g, dtype=torch.int32)
    blk[0, 0] = -1                                    # an empty slot: the block is not fetched, all its logits are -inf
    kernel = dsa.block_sparse_mqa_attn_return_logits(S, S_kv, bs, topk, H, D, block_N=8 if bs % 8 == 0 else 1)
    out = kernel(q.cuda(), k.cuda(), blk.cuda(), w.cuda(), ks.cuda(), ke.cuda()).cpu()
    check_status()
    # the CUDA-core kernel on the same inputs (the first case runs on the tensor cores by default)
    out_c = dsa.block_sparse_logits_raw(q.cuda(), k.cuda(), blk.cuda(), w.cuda(), ks.cuda(), ke.cuda(), bs, impl=1).cpu()
    assert torch.equal(torch.isinf(out), torch.isinf(out_c))
    torch.testing.assert_close(out[torch.isfinite(out)], out_c[torch.isfinite(out_c)], rtol=2e-5, atol=2e-4)
    ref = orc.block_sparse_logits(q, k, blk, bs, w, ks, ke)
    assert out.shape == ref.shape == (S, topk, bs)
    assert torch.equal(torch.isinf(out), torch.isinf(ref)), "masked positions differ"
    fin = torch.isfinite(ref)
    # products of 16-bit inputs are exact in fp32; only the summation order differs
    torch.testing.assert_close(out[fin], ref[fin], rtol=2e-5, atol=2e-4)


def test_block_sparse_logits_argument_checks():
    import tilelang_ascend_b200 as dsa
    with pytest.raises(AssertionError):
        dsa.block_sparse_mqa_attn_return_logits(8, 64, 16, 6, 4, 32)      # topk not divisible by 4
    kernel = dsa.block_sparse_mqa_attn_return_logits(8, 64, 16, 4, 4, 32)
    q = torch.zeros((8, 4, 32), dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        kernel(q, torch.zeros((64, 16), dtype=torch.float16, device="cuda"), torch.zeros((8, 4), dtype=torch.int32, device="cuda"),
               torch.zeros((8, 4), dtype=torch.float16, device="cuda"), torch.zeros(8, dtype=torch.int32, device="cuda"),
               torch.zeros(8, dtype=torch.int32, device="cuda"))


@pytest.mark.parametrize("B,S,H,D,bs,topk,maxb,nphys", [
    (2, 5, 32, 128, 128, 8, 20, 48),     # tensor-core kernel
    (3, 2, 12, 64, 32, 4, 9, 30),        # CUDA-core kernel
])
def test_paged_block_sparse_logits_match_oracle(B, S, H, D, bs, topk, maxb, nphys):
    import tilelang_ascend_b200 as dsa
    g = torch.Generator().manual_seed(B * 7 + S)
    q = (torch.rand((B, S, H, D), generator=g) - 0.5).to(torch.float16)
    cache = (torch.rand((nphys, bs, 1, D), generator=g) - 0.5).to(torch.float16)
    w = (torch.rand((B, S, H), generator=g) - 0.3).to(torch.float16)
    ctx = torch.randint(bs, maxb * bs, (B,), generator=g, dtype=torch.int32)
    bt = torch.stack([torch.randperm(nphys, generator=g)[:maxb] for _ in range(B)]).to(torch.int32)
    blk = torch.randint(0, maxb, (B, S, topk), generator=g, dtype=torch.int32)
    kernel = dsa.paged_block_sparse_mqa_attn_return_logits(B, S, nphys, bs, topk, H, D, maxb)
    out = kernel(q.view(B * S, H, D).cuda(), cache.cuda(), blk.view(B * S, topk).cuda(), w.view(B * S, H).cuda(), ctx.cuda(), bt.cuda()).cpu()
    check_status()
    ref = orc.paged_block_sparse_logits(q, cache, blk, bs, w, ctx, bt).reshape(B * S, topk, bs)
    assert torch.equal(torch.isinf(out), torch.isinf(ref)), "masked positions differ"
    fin = torch.isfinite(ref)
    torch.testing.assert_close(out[fin], ref[fin], rtol=2e-5, atol=2e-4)


@pytest.mark.parametrize("H,D,bs", [(32, 128, 128), (12, 64, 32)])
def test_paged_table_padding_is_never_dereferenced(H, D, bs):
    """Block-table entries past a sequence's context are padding (-1, as the reference's indexer front door writes them, or a
    number beyond the cache): logical blocks that lie wholly past the context must come back -inf on both kernels without the
    entry being used as an address, and blocks inside the context must be unaffected."""
    import tilelang_ascend_b200 as dsa
    B, S, topk, maxb, nphys = 2, 3, 8, 10, 24
    g = torch.Generator().manual_seed(H)
    q = (torch.rand((B, S, H, D), generator=g) - 0.5).to(torch.float16)
    cache = (torch.rand((nphys, bs, 1, D), generator=g) - 0.5).to(torch.float16)
    w = (torch.rand((B, S, H), generator=g) - 0.3).to(torch.float16)
    ctx = torch.tensor([3 * bs + 17, 6 * bs], dtype=torch.int32)
    bt = torch.stack([torch.randperm(nphys, generator=g)[:maxb] for _ in range(B)]).to(torch.int32)
    used = (ctx + bs - 1) // bs
    good = bt.clone()                      # oracle input: padding replaced by a valid block (its logits are masked anyway)
    for b in range(B):
        bt[b, int(used[b]):] = torch.tensor([-1, 1 << 20] * maxb)[: maxb - int(used[b])]
        good[b, int(used[b]):] = 0
    blk = torch.randint(0, maxb, (B, S, topk), generator=g, dtype=torch.int32)   # up to the batch-wide maximum, as the reference's test draws them
    ref = orc.paged_block_sparse_logits(q, cache, blk, bs, w, ctx, good).reshape(B * S, topk, bs)
    kernel = dsa.paged_block_sparse_mqa_attn_return_logits(B, S, nphys, bs, topk, H, D, maxb)
    args = (q.view(B * S, H, D).cuda(), cache.cuda(), blk.view(B * S, topk).cuda(), w.view(B * S, H).cuda(), ctx.cuda(), bt.cuda())
    out = kernel(*args).cpu()
    ke = ctx.repeat_interleave(S).contiguous().cuda()
    out_c = dsa.block_sparse_logits_raw(args[0], cache.view(nphys * bs, D).cuda(), args[2], args[3], torch.zeros_like(ke), ke, bs, impl=1,
                                        block_table=bt.cuda(), tokens_per_seq=S).cpu()
    check_status()
    past = (blk.view(B * S, topk) >= used.repeat_interleave(S)[:, None])
    assert past.any() and torch.isinf(out[past]).all() and torch.isinf(out_c[past]).all()
    for got in (out, out_c):
        assert torch.equal(torch.isinf(got), torch.isinf(ref)), "masked positions differ"
        fin = torch.isfinite(ref)
        torch.testing.assert_close(got[fin], ref[fin], rtol=2e-5, atol=2e-4)
