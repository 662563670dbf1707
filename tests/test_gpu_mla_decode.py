"""Dense MLA decode family (three factory signatures of examples_experiment/deepseek_mla/) on the GPU against the
reference-golden fixtures and the oracle, on the reference tests' own layered shapes."""
import math

import numpy as np
import pytest
import torch

import tilelang_ascend_b200 as dsa
from conftest import from_bits
from gpu_util import check_status
from oracle import dsa_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
H16 = torch.float16


def check_precision(actual: torch.Tensor, golden: torch.Tensor, what: str):
    """The reference tests' dual gate for fp16 (test_mla_decode.py:88-134): at least 99 % of the finite elements within
    atol 2^-14 + rtol 2^-9, and no element off by more than 0.1."""
    a, g = actual.float().cpu(), golden.float().cpu()
    fin = torch.isfinite(g)
    assert torch.equal(torch.isfinite(a), fin), f"{what}: non-finite pattern differs"
    err = (a[fin] - g[fin]).abs()
    ratio = float((err <= 2.0 ** -14 + 2.0 ** -9 * g[fin].abs()).float().mean())
    assert ratio >= 0.99 and float(err.max()) <= 0.1, f"{what}: matched ratio {ratio:.4f}, max abs err {float(err.max()):.3e}"


def gen(shape, kind, g):
    if kind == "randn":
        return torch.randn(shape, generator=g).half()
    lo, hi = kind
    return (torch.rand(shape, generator=g) * (hi - lo) + lo).half()


def test_mla_decode_matches_reference_golden_fixture(golden):
    g = golden("mla_decode.npz")
    q, q_pe, kv, k_pe = (from_bits(g[k], H16).to(DEV) for k in ("q", "q_pe", "kv", "k_pe"))
    B, H, D = q.shape
    out = dsa.mla_decode(B, H, 1, kv.shape[1], D, q_pe.shape[-1])(q, q_pe, kv, k_pe, torch.arange(128, device=DEV))
    check_precision(out, from_bits(g["out"], H16), "mla_decode vs ref_mla_decode fixture")
    check_status()


def test_persistent_variant_matches_reference_golden_fixture(golden):
    g = golden("mla_decode_persistent.npz")
    q, q_pe, kv, k_pe = (from_bits(g[k], H16).to(DEV) for k in ("q", "q_pe", "kv", "k_pe"))
    B, H, D = q.shape
    N, pe = kv.shape[1], q_pe.shape[-1]
    want = from_bits(g["out"], H16)
    out = dsa.flashattn_mla_decode(B, H, N, D, pe, 64, 64, 20)(q, q_pe, kv.view(B, N, D), k_pe.view(B, N, pe))
    check_precision(out, want, "flashattn_mla_decode vs fixture")
    check_precision(dsa.run_mla_decode(q, q_pe, kv, k_pe, 64, 64, 20), want, "run_mla_decode vs fixture")
    check_status()


def test_paged_variant_matches_reference_golden_fixture(golden):
    g = golden("mla_decode_paged.npz")
    q, pool = from_bits(g["q"], H16).to(DEV), from_bits(g["pool"], H16).to(DEV)
    bt = torch.from_numpy(g["block_table"]).to(DEV)
    bs, n = int(g["block_size"]), int(g["seqlen"])
    B, H = q.shape[:2]
    pad = bt.shape[1] * bs
    kernel = dsa.mla_decode_tilelang(B, H, 1, pad, 512, 64, 64, 32, bs, n, 20)
    out = kernel(q[..., :512].contiguous(), q[..., 512:].contiguous(), pool[..., :512].reshape(-1, 1, 512).contiguous(),
                 pool[..., 512:].reshape(-1, 1, 64).contiguous(), bt)
    check_precision(out, from_bits(g["out"], H16), "mla_decode_tilelang vs golden_mla_decode_paged fixture")
    check_status()


# (name, batch, heads, seqlen_kv, actual_seqlen_kv, value generator): the L0 / L1 cases of test_mla_decode.py:193-262
CASES = [
    ("l0_smoke", 1, 64, 128, None, "randn"),
    ("l0_standard", 1, 128, 8192, None, "randn"),
    ("l0_perf_target_8_of_132", 8, 128, 8192, None, "randn"),   # same per-sequence work, fewer sequences for the CPU oracle
    ("l1_aligned", 1, 64, 512, None, "randn"),
    ("l1_tail1", 1, 64, 640, 513, "randn"),
    ("l1_tailmid", 1, 64, 640, 576, "randn"),
    ("l1_prime", 1, 64, 512, 509, "randn"),
    ("l1_edge", 1, 64, 128, None, "randn"),
    ("l1_valrange_s", 1, 64, 512, None, (-1, 1)),
    ("l1_valrange_m", 1, 64, 512, None, (-10, 10)),
    ("l1_valrange_l", 1, 64, 512, None, (-50, 50)),
    ("l1_valrange_asym", 1, 64, 512, None, (-5, 10)),
]


@pytest.mark.parametrize("name,B,H,N,act,kind", CASES, ids=[c[0] for c in CASES])
def test_mla_decode_layered_cases(name, B, H, N, act, kind):
    g = torch.Generator().manual_seed(42)
    D, pe = 512, 64
    q, q_pe = gen((B, H, D), kind, g), gen((B, H, pe), kind, g)
    kv, k_pe = gen((B, N, 1, D), kind, g), gen((B, N, 1, pe), kind, g)
    n = N if act is None else act
    want = orc.mla_decode(q, q_pe, kv[:, :n], k_pe[:, :n])
    kernel = dsa.mla_decode(B, H, 1, N, D, pe, actual_seqlen_kv=-1 if act is None else act)
    out = kernel(q.to(DEV), q_pe.to(DEV), kv.to(DEV), k_pe.to(DEV), torch.arange(128, device=DEV))
    check_precision(out, want.half(), name)
    if act is None:   # the persistent signature computes the same thing from 3-D caches
        out2 = dsa.flashattn_mla_decode(B, H, N, D, pe, 64, 64, 20)(q.to(DEV), q_pe.to(DEV), kv.view(B, N, D).to(DEV), k_pe.view(B, N, pe).to(DEV))
        assert torch.equal(out2, out)
    check_status()


# (name, batch, cache_seqlen, block_size, scale override, value scale): cases of test_mla_decode_paged.py:173-275
PAGED = [
    ("l0_small_b2", 2, 256, 256, None, 1.0),
    ("l0_seq2048", 4, 2048, 256, None, 1.0),
    ("l1_tail_1", 1, 65, 256, None, 1.0),
    ("l1_tail_mid", 2, 160, 256, None, 1.0),
    ("l1_prime", 1, 97, 256, None, 1.0),
    ("l1_param_bs512", 1, 512, 512, None, 1.0),
    ("l1_param_scale", 1, 256, 256, 0.05, 1.0),
    ("l1_valrange_s", 1, 256, 256, None, 0.25),
    ("b_single_token", 1, 1, 256, None, 1.0),
]


@pytest.mark.parametrize("name,B,n,bs,scale,vs", PAGED, ids=[c[0] for c in PAGED])
def test_mla_decode_paged_cases(name, B, n, bs, scale, vs):
    g = torch.Generator().manual_seed(42)
    H, dv, dpe = 128, 512, 64
    pad = max(math.ceil(n / bs) * bs, 256)
    nb = pad // bs
    pre = (dv + dpe) ** -0.5 if scale is None else scale
    qf = ((torch.randn((B, H, dv + dpe), generator=g) * vs).half() * pre).half()    # the caller folds the softmax scale into Q
    pool = (torch.randn((B * nb, bs, 1, dv + dpe), generator=g) * vs).half()
    bt = torch.randperm(B * nb, generator=g).to(torch.int32).view(B, nb)            # scattered physical blocks
    q, q_pe = qf[..., :dv].contiguous(), qf[..., dv:].contiguous()
    kvp, kpp = pool[..., :dv].reshape(-1, 1, dv).contiguous(), pool[..., dv:].reshape(-1, 1, dpe).contiguous()
    want = orc.mla_decode_paged(q, q_pe, kvp, kpp, bt, [n] * B, bs, softmax_scale=1.0)
    kernel = dsa.mla_decode_tilelang(B, H, 1, pad, dv, dpe, 256, 32, bs, n, 20, pre)
    out = kernel(q.to(DEV), q_pe.to(DEV), kvp.to(DEV), kpp.to(DEV), bt.to(DEV))
    check_precision(out, want.half(), name)
    check_status()


def test_argument_rules():
    with pytest.raises(ValueError, match="at most"):
        dsa.mla_decode(1, 128, 1, 16384, 512, 64)
    with pytest.raises(AssertionError):
        dsa.mla_decode_tilelang(1, 128, 2, 256, 512, 64, 256, 32, 256, 256, 20)
    with pytest.raises(AssertionError):
        dsa.mla_decode_tilelang(1, 128, 1, 256, 512, 64, 256, 32, 256, 300, 20)
    q = torch.zeros((1, 64, 512), dtype=H16, device=DEV)
    with pytest.raises(ValueError, match="dtype"):
        dsa.mla_decode(1, 64, 1, 128, 512, 64)(q, torch.zeros((1, 64, 64), dtype=torch.bfloat16, device=DEV),
                                               torch.zeros((1, 128, 1, 512), dtype=H16, device=DEV), torch.zeros((1, 128, 1, 64), dtype=H16, device=DEV))
    with pytest.raises(ValueError, match="shapes"):
        dsa.mla_decode(1, 64, 1, 128, 512, 64)(q, torch.zeros((1, 64, 64), dtype=H16, device=DEV),
                                               torch.zeros((1, 64, 1, 512), dtype=H16, device=DEV), torch.zeros((1, 64, 1, 64), dtype=H16, device=DEV))
