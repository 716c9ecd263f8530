"""The oracle held to the reference's own code through the committed fixtures
(tests/golden/make_golden.py made them by running the reference's _attn_ref.py,
merge_splits and switches.py in the build container)."""

import json
import math
import os

import torch

from oracle import paged_oracle as orc

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_decode_oracle_equals_the_references_float64_softmax():
    g = torch.load(os.path.join(GOLD, "attn_golden.pt"))
    got = orc.paged_decode_ref(g["q"], g["k"].transpose(1, 2), g["v"].transpose(1, 2), g["table"], g["lens"])
    assert torch.equal(got, g["out"]) or (got - g["out"]).abs().max().item() < 1e-6
    fp32 = orc.paged_decode_ref_fp32(g["q"], g["k"].transpose(1, 2), g["v"].transpose(1, 2), g["table"], g["lens"])
    assert (fp32 - g["out"]).abs().max().item() < 1e-5


def test_prefill_oracle_equals_the_references_masked_softmax():
    g = torch.load(os.path.join(GOLD, "attn_golden.pt"))
    got = orc.paged_prefill_ref(g["prefill_q"], g["k"].transpose(1, 2), g["v"].transpose(1, 2), g["table"], g["lens"],
                                g["prefill_q_start"])
    assert (got - g["prefill_out"]).abs().max().item() < 1e-6


def test_tolerance_functions_equal_the_references():
    g = torch.load(os.path.join(GOLD, "attn_golden.pt"))
    assert orc.ULPS == g["ULPS"] and orc.TOL == g["TOL"]
    assert math.isclose(orc.rel(g["noisy"], g["out"]), g["rel"], rel_tol=1e-6)
    assert math.isclose(orc.ulps(g["noisy"], g["out"]), g["ulps"], rel_tol=1e-6)


def test_merge_restatement_equals_the_references_merge_splits():
    g = torch.load(os.path.join(GOLD, "merge_golden.pt"))
    out = torch.empty_like(g["out"])
    orc.merge_splits_unnormalised(g["o_part"], g["ml_part"], g["splits"], out)
    assert torch.equal(out, g["out"])


def test_lse_convention_gives_the_same_answer_as_the_references_merge():
    """This build keeps normalised partials + natural-log lse; converting the reference's
    (unnormalised numerators, (m, l) in log2) to it and folding must give the reference's answer."""
    g = torch.load(os.path.join(GOLD, "merge_golden.pt"))
    o, ml, s = g["o_part"], g["ml_part"], g["splits"]
    rs, hkv, tile, d = o.shape
    reqs = rs // s
    ml_t = ml.permute(0, 1, 3, 2)                                   # (rows, hkv, tile, 2)
    po, lse = orc.to_lse_convention(o.reshape(rs, hkv * tile, d), ml_t.reshape(rs, hkv * tile, 2))
    po = po.view(reqs, s, hkv * tile, d).transpose(0, 1).contiguous()
    lse = lse.view(reqs, s, hkv * tile).transpose(0, 1).contiguous()
    got, _ = orc.merge_lse_ref(po, lse)
    assert (got.view(reqs, hkv, tile, d) - g["out"]).abs().max().item() < 1e-5


def test_split_partials_fold_back_to_the_unsplit_answer():
    g = torch.load(os.path.join(GOLD, "attn_golden.pt"))
    q, k, v, table, lens = g["q"], g["k"], g["v"], g["table"], g["lens"]
    page, hkv, d = k.shape[2], k.shape[1], k.shape[3]
    group = q.shape[1] // hkv
    cuts = 3
    parts_o = torch.zeros(cuts, len(lens), q.shape[1], d)
    parts_l = torch.full((cuts, len(lens), q.shape[1]), float("-inf"))
    for i, s in enumerate(lens.tolist()):
        pages = table[i, : -(-s // page)].long()
        kk = k[pages].transpose(1, 2).reshape(-1, hkv, d)[:s]
        vv = v[pages].transpose(1, 2).reshape(-1, hkv, d)[:s]
        per = -(-s // cuts)
        for c in range(cuts):
            lo, hi = min(s, c * per), min(s, (c + 1) * per)
            for kh in range(hkv):
                hs = slice(kh * group, (kh + 1) * group)
                parts_o[c, i, hs], parts_l[c, i, hs] = orc.partial_ref(q[i, hs], kk[lo:hi, kh], vv[lo:hi, kh], d ** -0.5)
    poison = parts_o.clone()
    poison[torch.isinf(parts_l)] = float("nan")          # an empty part's memory may hold anything
    got, _ = orc.merge_lse_ref(poison, parts_l)
    assert (got - g["out"]).abs().max().item() < 1e-5


def test_fp8_quantise_saturates_and_rounds_to_nearest_even():
    sc = torch.tensor([0.5])
    x = torch.tensor([1e4, -1e4, 224.0, 0.0, 0.03125, 8.5, 9.5, 232.0])
    q = orc.quantize_fp8(x, sc)
    back = q.float()
    assert back[0] == 448 and back[1] == -448 and back[2] == 448 and back[3] == 0
    assert torch.isfinite(back).all()
    # 17 and 19 sit halfway between e4m3 neighbours (16, 18, 20): ties go to the even mantissa
    assert back[5] == 16.0 and back[6] == 20.0
    assert orc.dequantize_fp8(q, sc)[2] == 224.0


def test_switch_goldens_cover_both_routes():
    rows = json.load(open(os.path.join(GOLD, "switches_golden.json")))["rows"]
    assert {r["route"] for r in rows} == {"vllm_backend", "vllm_prefill"} and len(rows) > 200
