"""The in-engine A/B harness's verdict arithmetic (no engine needed): best of rounds, ratio to
stock, a noise band from the rounds themselves -- the reference's rule that a gap inside
max(2 %, the noise) is not a result (python/hk/integration/ab.py:17-21)."""

import pytest

from hk_dsl_b200.integration import ab


def _round(total, short, prefill):
    return {"1024x16": {"total": total, "short": short, "prefill": prefill, "tokens": [1, 2, 3]}, "_startup_s": 1.0}


def test_verdicts():
    assert ab.verdict(1.10, 0.02) == "win"
    assert ab.verdict(0.90, 0.02) == "loss"
    assert ab.verdict(1.01, 0.02) == "tie"
    assert ab.verdict(1.05, 0.08) == "noise"


def test_judge_takes_best_of_rounds_and_the_widest_spread_as_band():
    rounds = {"stock": [_round(1.00, 0.40, 0.10), _round(1.04, 0.42, 0.10)],
              "hk": [_round(0.80, 0.36, 0.10), _round(0.82, 0.36, 0.11)]}
    rows = {(r["metric"], r["arm"]): r for r in ab.judge(rounds, tokens=96, short=32)}
    total = rows[("total", "hk")]
    assert total["ms"] == pytest.approx(800.0) and total["stock_ms"] == pytest.approx(1000.0)
    assert total["ratio"] == pytest.approx(1.25) and total["band"] == pytest.approx(0.04) and total["verdict"] == "win"
    dec = rows[("decode", "hk")]
    assert dec["stock_ms"] == pytest.approx((1.00 - 0.40) / 64 * 1e3) and dec["ms"] == pytest.approx((0.80 - 0.36) / 64 * 1e3)
    pre = rows[("prefill", "hk")]
    assert pre["ratio"] == pytest.approx(1.0) and pre["band"] == pytest.approx(0.10) and pre["verdict"] == "noise"
    assert ("total", "stock") not in rows


def test_shapes_are_gqa_models():
    for hidden, hq, hkv, d, inter, vocab in ab.SHAPES.values():
        assert hq % hkv == 0 and d == 128
