"""Generate the golden fixtures in this folder from the reference's own CPU goldens.

Run where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/tilelang-ascend

Only the named golden *functions* are taken from the reference files: each file is parsed with
``ast`` and the wanted ``FunctionDef`` nodes (plus the helpers they call) are compiled on their own,
so no reference module body -- which would need an NPU -- is executed, and no reference source is
copied into this repository.  The fixtures hold seeded inputs and the reference outputs; bf16
tensors are stored as their uint16 bit patterns.
"""
from __future__ import annotations

import argparse
import ast
import math
import os
import sys
from typing import Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def load_functions(path: str, names: Sequence[str], extra_globals: Optional[dict] = None) -> dict:
    """Compile only the FunctionDef / simple constant assignments called ``names`` from ``path``."""
    with open(path, "r", encoding="utf-8") as fh:
        tree = ast.parse(fh.read(), filename=path)
    keep = []
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            keep.append(node)
        elif isinstance(node, ast.Assign) and len(node.targets) == 1 and isinstance(node.targets[0], ast.Name) \
                and node.targets[0].id in names:
            keep.append(node)
    found = {n.name if isinstance(n, ast.FunctionDef) else n.targets[0].id for n in keep}
    missing = set(names) - found
    if missing:
        raise RuntimeError(f"{path}: missing {sorted(missing)}")
    mod = ast.Module(body=keep, type_ignores=[])
    env = {"torch": torch, "np": np, "math": math, "F": F, "Optional": Optional, "Tuple": Tuple,
           "Sequence": Sequence}
    if extra_globals:
        env.update(extra_globals)
    exec(compile(mod, path, "exec"), env)
    return env


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16/fp16 tensor -> uint16 bit pattern; everything else -> numpy as is."""
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("DSA_REFERENCE_ROOT"),
                    help="root of a checkout of the reference project (or set DSA_REFERENCE_ROOT)")
    args = ap.parse_args()
    ref = args.reference
    if not ref or not os.path.isdir(ref):
        raise SystemExit("give the reference checkout with --reference or DSA_REFERENCE_ROOT")
    sys.path.insert(0, os.path.join(HERE, "..", ".."))
    from oracle import dsa_oracle as orc

    # ---- sparse MLA forward (bf16 variant of the torch golden) ------------------------------
    env = load_functions(
        os.path.join(ref, "examples/sparse_flash_attention/example_sparse_flash_attn_dynamic_shape.py"),
        ["ref_sparse_attention_fwd_interface"])
    fwd_golden = env["ref_sparse_attention_fwd_interface"]
    for tag, (B, S, S_kv, H, topk, seed) in {
        "a": (2, 8, 64, 16, 16, 0),      # padding present (early queries see < topk keys)
        "b": (1, 4, 256, 128, 64, 1),    # 128 heads, no padding
    }.items():
        q, kv, idx = orc.make_sparse_mla_inputs(B, S, S_kv, H, topk, seed=seed, causal=True, pad=-1)
        if tag == "a":  # let early queries see few keys: start the query block at position 5
            q_start = 5
            rng = np.random.default_rng(7)
            idx = torch.full((B, S, 1, topk), -1, dtype=torch.int32)
            for b in range(B):
                for t in range(S):
                    n = q_start + t + 1
                    sel = rng.permutation(n)[:topk]
                    idx[b, t, 0, : len(sel)] = torch.from_numpy(sel.astype(np.int32))
            # two slots beyond the causal limit: the golden must mask them
            idx[0, 0, 0, topk - 1] = 40
            idx[1, 3, 0, topk - 1] = 63
        else:
            q_start = S_kv - S
        idx_ref = torch.where(idx < 0, torch.full_like(idx, S_kv), idx)  # golden's sentinel is S_kv
        out = fwd_golden(q, kv, idx_ref, q_start, kv_stride=1)
        np.savez_compressed(os.path.join(HERE, f"sparse_mla_fwd_{tag}.npz"), q=bits(q), kv=bits(kv),
                            indices=idx.numpy(), q_start=np.int64(q_start), out=bits(out))

    # ---- NumPy golden of the paged / decode wrapper (BSND, block size 1, -1 terminated) ------
    env = load_functions(os.path.join(ref, "examples/sparse_flash_attention/sfa_golden.py"),
                         ["pa_to_bsnd", "trans_tnd_actseq", "trans_tnd_to_bsnd", "trans_bnsd_to_tnd", "gather_kv",
                          "mask", "softmax", "cpu_sparse_flash_attention"])
    sfa = env["cpu_sparse_flash_attention"]
    B, S, S_kv, H, topk = 2, 3, 96, 16, 24
    q, kv, _ = orc.make_sparse_mla_inputs(B, S, S_kv, H, topk, seed=3)
    act_q = np.array([3, 2], dtype=np.int64)
    act_kv = np.array([96, 50], dtype=np.int64)
    rng = np.random.default_rng(11)
    idx = np.full((B, S, 1, topk), -1, dtype=np.int32)
    for b in range(B):
        for t in range(int(act_q[b])):
            n = int(act_kv[b] - act_q[b] + t + 1)
            sel = rng.permutation(n)[: min(topk, n) - (1 if t == 0 else 0)]  # one row ends early with -1
            idx[b, t, 0, : len(sel)] = sel
    out = sfa(q[..., :512], kv[..., :512], None, torch.from_numpy(idx), 576 ** -0.5, 1,
              torch.from_numpy(act_q), torch.from_numpy(act_kv), query_rope=q[..., 512:], key_rope=kv[..., 512:],
              layout_query="BSND", layout_kv="BSND", sparse_mode=3)
    np.savez_compressed(os.path.join(HERE, "sfa_numpy_golden.npz"), q=bits(q), kv=bits(kv), indices=idx,
                        act_q=act_q, act_kv=act_kv, out=np.asarray(out, dtype=np.float32))

    # ---- LSE definition (V4 golden with the sink switched off) ---------------------------------
    env = load_functions(os.path.join(ref, "examples/deepseek_v4/sparse_flash_mla/sparse_flash_mla_golden.py"),
                         ["GOLDEN_S2_TILE", "_gather_cmp_kv_tokens", "sparse_flash_mla_golden_bnsd"])
    v4 = env["sparse_flash_mla_golden_bnsd"]
    g = torch.Generator().manual_seed(5)
    B, N1, S1, S2, D = 1, 8, 6, 40, 64
    qb = torch.randn((B, N1, S1, D), generator=g).to(torch.bfloat16)
    kb = torch.randn((B, 1, S2, D), generator=g).to(torch.bfloat16)
    sinks = torch.full((N1,), float("-inf"))
    win = 15
    o, lse = v4(qb, kb, sinks, act_q_lens=[S1], act_kv_lens=[S2], softmax_scale=D ** -0.5, ori_win_left=win,
                return_lse=True)
    np.savez_compressed(os.path.join(HERE, "lse_window.npz"), q=bits(qb), k=bits(kb), win=np.int64(win),
                        out=bits(o), lse=lse.numpy())

    # ---- V4 sparse_flash_mla: window + selected / all compressed tokens + sinks ------------------
    g = torch.Generator().manual_seed(9)
    B, N1, S1, S2, D, K, ratio, win = 2, 8, 6, 41, 64, 8, 4, 7
    qb = torch.randn((B, N1, S1, D), generator=g).to(torch.bfloat16)
    kb = torch.randn((B, 1, S2, D), generator=g).to(torch.bfloat16)
    cb = torch.randn((B, 1, S2 // ratio, D), generator=g).to(torch.bfloat16)
    sinks = torch.randn((N1,), generator=g)
    act_q, act_kv = [6, 4], [41, 30]
    rng = np.random.default_rng(4)
    ci = np.full((B, S1, 1, K), -1, dtype=np.int32)
    for b in range(B):
        for s_ in range(act_q[b]):
            n = rng.integers(0, K + 1)
            ci[b, s_, 0, :n] = rng.integers(0, S2 // ratio, size=n)   # includes entries at / above the threshold and repeats
    o3, l3 = v4(qb, kb, sinks, act_q_lens=act_q, act_kv_lens=act_kv, softmax_scale=D ** -0.5, cmp_k_bnsd=cb,
                cmp_sparse_indices=torch.from_numpy(ci), cmp_ratio=ratio, ori_win_left=win, return_lse=True)
    o2, l2 = v4(qb, kb, sinks, act_q_lens=act_q, act_kv_lens=act_kv, softmax_scale=D ** -0.5, cmp_k_bnsd=cb,
                cmp_ratio=ratio, ori_win_left=win, return_lse=True)
    o1, l1 = v4(qb, kb, sinks, act_q_lens=act_q, act_kv_lens=act_kv, softmax_scale=D ** -0.5, ori_win_left=win, return_lse=True)
    np.savez_compressed(os.path.join(HERE, "sparse_flash_mla_v4.npz"), q=bits(qb), k=bits(kb), c=bits(cb), sinks=sinks.numpy(),
                        act_q=np.array(act_q), act_kv=np.array(act_kv), ci=ci, ratio=np.int64(ratio), win=np.int64(win),
                        out3=bits(o3), lse3=l3.numpy(), out2=bits(o2), lse2=l2.numpy(), out1=bits(o1), lse1=l1.numpy())

    # ---- HISA block-sparse indexer logits ---------------------------------------------------------
    env = load_functions(os.path.join(ref, "examples/HISA/block_sparse_mqa_attn_expert_test.py"), ["ref_block_sparse_mqa_attn"])
    g = torch.Generator().manual_seed(21)
    S, S_kv, H, D, bs, topk = 12, 256, 8, 32, 16, 4
    qh = torch.rand((S, H, D), generator=g).to(torch.float16) - 0.5
    kh = torch.rand((S_kv, D), generator=g).to(torch.float16) - 0.5
    wh = (torch.rand((S, H), generator=g) - 0.3).to(torch.float16)
    ks_ = torch.randint(0, 40, (S,), generator=g, dtype=torch.int32)
    ke_ = (torch.arange(1, S + 1, dtype=torch.int32) * (S_kv // S)).clamp(max=S_kv)
    blk = torch.randint(0, S_kv // bs, (S, topk), generator=g, dtype=torch.int32)
    hl = env["ref_block_sparse_mqa_attn"](qh, kh, blk, bs, wh, ks_, ke_)
    np.savez_compressed(os.path.join(HERE, "hisa_block_sparse_logits.npz"), q=bits(qh), k=bits(kh), w=bits(wh), ks=ks_.numpy(), ke=ke_.numpy(),
                        blk=blk.numpy(), bs=np.int64(bs), logits=hl.numpy())

    env = load_functions(os.path.join(ref, "examples/HISA/paged_block_sparse_mqa_attn_expert.py"), ["ref_paged_block_sparse_mqa_attn"])
    g = torch.Generator().manual_seed(22)
    B, S, H, D, bs, topk, maxb, nphys = 2, 3, 8, 32, 16, 4, 6, 14
    qp = torch.rand((B, S, H, D), generator=g).to(torch.float16) - 0.5
    cache = torch.rand((nphys, bs, 1, D), generator=g).to(torch.float16) - 0.5
    wp = (torch.rand((B, S, H), generator=g) - 0.3).to(torch.float16)
    ctx = torch.tensor([70, 41], dtype=torch.int32)
    bt = torch.stack([torch.randperm(nphys, generator=g)[:maxb] for _ in range(B)]).to(torch.int32)
    blkp = torch.randint(0, maxb, (B, S, topk), generator=g, dtype=torch.int32)
    pl = env["ref_paged_block_sparse_mqa_attn"](qp, cache, blkp, bs, wp, ctx, bt)
    np.savez_compressed(os.path.join(HERE, "hisa_paged_logits.npz"), q=bits(qp), cache=bits(cache), w=bits(wp), ctx=ctx.numpy(), bt=bt.numpy(),
                        blk=blkp.numpy(), bs=np.int64(bs), logits=pl.numpy())

    # ---- lightning indexer, production golden ---------------------------------------------------
    env = load_functions(os.path.join(ref, "examples/deepseek_v4/lightning_indexer.py"),
                         ["_NEG_INF", "cpu_lightning_indexer"])
    li = env["cpu_lightning_indexer"]
    cases = {}
    for tag, (B, S1, S2, N1, K, mode, aq, ak, seed) in {
        "causal": (2, 12, 300, 16, 64, 3, [12, 7], [300, 129], 0),   # rows with fewer than K keys, ragged batch
        "full": (1, 5, 200, 64, 32, 0, [5], [200], 1),
        "ties": (1, 6, 96, 4, 48, 3, [6], [96], 2),
    }.items():
        q, k, w = orc.make_indexer_inputs(B, S1, S2, N1, 128, seed=seed)
        if tag == "ties":  # repeated key rows give exactly equal scores: the tie rule decides
            k[:, 1::2] = k[:, 0::2]
        idx, scores, val = li(q, k, w, actual_seq_lengths_query=torch.tensor(aq), actual_seq_lengths_key=torch.tensor(ak),
                              sparse_count=K, sparse_mode=mode)
        cases.update({f"{tag}_q": bits(q), f"{tag}_k": bits(k), f"{tag}_w": w.numpy(), f"{tag}_aq": np.array(aq),
                      f"{tag}_ak": np.array(ak), f"{tag}_mode": np.int64(mode), f"{tag}_K": np.int64(K),
                      f"{tag}_idx": idx.numpy(), f"{tag}_scores": scores.numpy(), f"{tag}_val": bits(val)})
    np.savez_compressed(os.path.join(HERE, "lightning_indexer.npz"), **cases)

    # ---- simple indexer golden (fp16 einsum + torch.topk) ---------------------------------------
    B, N2, G, S1, S2, D, TOP_K = 1, 1, 4, 8, 128, 64, 16
    env = load_functions(os.path.join(ref, "examples/lightning_indexer/example_lightning_indexer.py"), ["index_golden"],
                         {"TOP_K": TOP_K})
    g = torch.Generator().manual_seed(2)
    q = torch.randn((B, S1, N2, G, D), generator=g).half()
    k = torch.randn((B, S2, N2, D), generator=g).half()
    w = torch.randn((B, S1, N2, G, 1), generator=g).float()
    qk, gi = env["index_golden"](q, k, w)
    np.savez_compressed(os.path.join(HERE, "simple_indexer.npz"), q=bits(q), k=bits(k), w=w.numpy(), qk=qk.numpy(),
                        indices=gi.numpy())

    # ---- stand-alone selector ---------------------------------------------------------------------
    env = load_functions(os.path.join(ref, "examples/topk_selector/example_topk_selector.py"), ["ref_program"])
    g = torch.Generator().manual_seed(0)
    x = torch.randn((12, 1000), generator=g)
    np.savez_compressed(os.path.join(HERE, "topk_selector.npz"), x=x.numpy(),
                        indices=env["ref_program"](x, 100).numpy().astype(np.int32))

    # ---- dense MLA decode ----------------------------------------------------------------------------
    env = load_functions(os.path.join(ref, "examples_experiment/deepseek_mla/example_mla_decode/test_mla_decode.py"),
                         ["ref_mla_decode"])
    g = torch.Generator().manual_seed(4)
    B, H, N, D, pe = 2, 16, 200, 512, 64
    q = torch.randn((B, H, D), generator=g).half()
    q_pe = torch.randn((B, H, pe), generator=g).half()
    kv = torch.randn((B, N, 1, D), generator=g).half()
    k_pe = torch.randn((B, N, 1, pe), generator=g).half()
    out = env["ref_mla_decode"](q, q_pe, kv, k_pe)
    np.savez_compressed(os.path.join(HERE, "mla_decode.npz"), q=bits(q), q_pe=bits(q_pe), kv=bits(kv), k_pe=bits(k_pe),
                        out=bits(out))
    # ---- dense MLA decode, paged cache (the caller pre-scales Q; the golden is called with scale 1) -----
    env = load_functions(os.path.join(ref, "examples_experiment/deepseek_mla/example_mla_decode_paged/test_mla_decode_paged.py"),
                         ["golden_mla_decode_paged"])
    g = torch.Generator().manual_seed(6)
    B, H, dv, dpe, bs, nblk = 2, 16, 512, 64, 64, 3
    seqlens = torch.tensor([150, 150], dtype=torch.int32)   # a tail inside the third block
    qf = (torch.randn((B, H, dv + dpe), generator=g) * (dv + dpe) ** -0.5).half()
    pool = torch.randn((B * nblk, bs, 1, dv + dpe), generator=g).half()
    btp = torch.randperm(B * nblk, generator=g).to(torch.int32).view(B, nblk)
    kvp = pool[..., :dv].reshape(-1, 1, dv).contiguous()
    kpp = pool[..., dv:].reshape(-1, 1, dpe).contiguous()
    outp = env["golden_mla_decode_paged"](qf[..., :dv].contiguous(), qf[..., dv:].contiguous(), kvp, kpp, btp, seqlens, B, H, 1, dv, dpe,
                                          bs, nblk * bs, softmax_scale=1.0)
    np.savez_compressed(os.path.join(HERE, "mla_decode_paged.npz"), q=bits(qf), pool=bits(pool), block_table=btp.numpy(),
                        seqlen=np.int64(150), block_size=np.int64(bs), out=bits(outp))

    # ---- dense MLA decode, persistent variant's golden (einops path when einops is importable, as in the reference) -----
    try:
        from einops import einsum as _einsum, rearrange as _rearrange
    except ImportError:
        _einsum = _rearrange = None
    env = load_functions(os.path.join(ref, "examples_experiment/deepseek_mla/example_mla_decode_persistent/test_mla_decode_persistent.py"),
                         ["ref_mla_decode"], {"rearrange": _rearrange, "einsum": _einsum})
    g = torch.Generator().manual_seed(8)
    B, H, N, D, pe = 2, 64, 192, 512, 64
    q = torch.randn((B, H, D), generator=g).half()
    q_pe = torch.randn((B, H, pe), generator=g).half()
    kv = torch.randn((B, N, 1, D), generator=g).half()
    k_pe = torch.randn((B, N, 1, pe), generator=g).half()
    out = env["ref_mla_decode"](q, q_pe, kv, k_pe)
    np.savez_compressed(os.path.join(HERE, "mla_decode_persistent.npz"), q=bits(q), q_pe=bits(q_pe), kv=bits(kv), k_pe=bits(k_pe),
                        out=bits(out))
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
