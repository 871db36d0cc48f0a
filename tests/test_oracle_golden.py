"""The CPU oracle against fixtures produced by the reference's own code.

Integer tables must match bit for bit; float results within 1e-5 (both sides
are float32 on the CPU)."""

from __future__ import annotations

import os

import numpy as np
import pytest
import torch

import natten_oracle as oracle
from conftest import GOLDEN, tup
from make_golden import CASES, make_inputs, window_grid

TOL = dict(atol=2e-5, rtol=2e-5)


def test_window_tables_bit_exact():
    t = np.load(os.path.join(GOLDEN, "window_tables.npz"))
    grid = t["grid"]
    assert [tuple(int(v) for v in g) for g in grid] == list(window_grid())
    for (length, k, d), off in zip(grid, t["offsets"]):
        length, k, d = int(length), int(k), int(d)
        pos = range(length)
        starts = [oracle.window_start(p, length, k, d) for p in pos]
        assert starts == t["starts"][off:off + length].tolist(), (length, k, d)
        assert [oracle.window_end(s, length, k, d) for s in starts] == t["ends"][off:off + length].tolist()
        assert [oracle.pb_start(p, length, k, d) for p in pos] == t["pb_starts"][off:off + length].tolist()
        # the dilation-group formula of the allin1 helpers is the same function for odd kernels
        if k % 2 == 1:
            assert t["grouped_starts"][off:off + length].tolist() == starts
            assert [oracle.window_start_grouped(p, length, k, d) for p in pos] == starts


def test_known_answers_from_reference_tests():
    # tests/test_shift_semantics.py:53-64 of the reference: L=32, K=3, last position, dilation 1
    assert oracle.window_start(31, 32, 3, 1) == 29
    assert oracle.pb_start(31, 32, 3, 1) == 0
    # phase alignment under dilation and bounds (tests/test_shift_semantics.py:11-50)
    for length, k, d in [(33, 7, 4), (20, 5, 3), (17, 3, 5)]:
        for p in range(length):
            s = oracle.window_start(p, length, k, d)
            assert s % d == p % d and 0 <= s and s + (k - 1) * d < length
            assert 0 <= oracle.pb_start(p, length, k, d) <= k - 1


def test_index_tables_bit_exact():
    t = np.load(os.path.join(GOLDEN, "index_tables.npz"))
    off = 0
    for length, k, d, stride, causal, n in t["axis_cases"]:
        idx, ok = oracle.axis_table(oracle.query_positions(int(length), int(stride)), int(length), int(k), int(d), bool(causal))
        m = int(n) * int(k)
        assert idx.reshape(-1).tolist() == t["axis_idx"][off:off + m].tolist()
        assert ok.reshape(-1).tolist() == t["axis_ok"][off:off + m].tolist()
        off += m
    lin, ok, _ = oracle.neighbor_tables((7, 9), (3, 5), (1, 1), (2, 1), (True, False))
    assert np.array_equal(lin, t["lin2"]) and np.array_equal(ok, t["ok2"])
    lin, ok, _ = oracle.neighbor_tables((4, 5, 6), (3, 3, 5), (1, 1, 1), (1, 1, 1), (False, True, False))
    assert np.array_equal(lin, t["lin3"]) and np.array_equal(ok, t["ok3"])


def _close(got, want, name):
    got = got.detach().numpy() if torch.is_tensor(got) else got
    assert got.shape == want.shape, (name, got.shape, want.shape)
    assert np.array_equal(np.isinf(got), np.isinf(want)), f"{name}: -inf pattern differs"
    fin = np.isfinite(want)
    np.testing.assert_allclose(got[fin], want[fin], err_msg=name, **TOL)


@pytest.mark.parametrize("idx", range(len(CASES)))
def test_pure_cases(idx, golden_cases):
    cases, ref = golden_cases
    case = cases[idx]
    import json
    assert case == json.loads(json.dumps(CASES[idx]))
    x = {k: torch.from_numpy(v) for k, v in make_inputs(idx, case).items()}
    rank = len(case["shape"]) - 3
    ks, st = tup(case["kernel_size"], rank), tup(case["stride"], rank)
    dl, ca = tup(case["dilation"], rank), tup(case["is_causal"], rank)
    kind = case["kind"]
    g = lambda name: ref[f"c{idx}_{name}"]
    if kind == "fused":
        out, grads = oracle.grads(lambda q, k, v: oracle.na(q, k, v, ks, st, dl, ca), [x["q"], x["k"], x["v"]], x["cot"])
        _close(out, g("out"), "out")
        for name, t in zip(("dq", "dk", "dv"), grads):
            _close(t, g(name), name)
    elif kind == "qk":
        out = oracle.na_qk(x["q"], x["k"], ks, st, dl, ca)
        _close(out, g("out"), "logits")
        fin = lambda q, k: torch.nan_to_num(oracle.na_qk(q, k, ks, st, dl, ca), neginf=0.0)
        _, grads = oracle.grads(fin, [x["q"], x["k"]], torch.where(torch.isinf(out), torch.zeros_like(x["cot"]), x["cot"]))
        _close(grads[0], g("dq"), "dq")
        _close(grads[1], g("dk"), "dk")
    elif kind == "av":
        out, grads = oracle.grads(lambda a, v: oracle.na_av(a, v, ks, st, dl, ca), [x["attn"], x["v"]], x["cot"])
        _close(out, g("out"), "out")
        _close(grads[0], g("dattn"), "dattn")
        _close(grads[1], g("dv"), "dv")
    elif kind == "lse_extra":
        names = ["q", "k", "v"] + (["ak", "av"] if "ak" in x else [])
        def fn(*a):
            kw = dict(additional_keys=a[3], additional_values=a[4]) if len(a) == 5 else {}
            return oracle.na(a[0], a[1], a[2], ks, st, dl, ca, return_lse=True, **kw)
        (out, lse), grads = oracle.grads(fn, [x[n] for n in names], (x["cot"], x["cot_lse"]))
        _close(out, g("out"), "out")
        _close(lse, g("lse"), "lse")
        for n, t in zip(names, grads):
            _close(t, g("d" + n), "d" + n)
    elif kind == "varlen":
        fn = lambda q, k, v: oracle.na_varlen(q, k, v, case["sizes"], ks, dl)
        out, grads = oracle.grads(fn, [x["q"], x["k"], x["v"]], x["cot"])
        _close(out, g("out"), "out")
        for name, t in zip(("dq", "dk", "dv"), grads):
            _close(t, g(name), name)
    elif kind == "merge":
        n = case["n_parts"]
        out, lse = oracle.merge_attentions([x[f"o{j}"] for j in range(n)], [x[f"l{j}"] for j in range(n)])
        _close(out, g("out"), "out")
        _close(lse, g("lse"), "lse")
    elif kind == "qk_rpb":
        _close(oracle.qk_rpb(x["q"], x["k"], x.get("rpb"), case["kernel_size"], case["dilation"], 0.288), g("out"), "logits")
    elif kind == "av_fused":
        _close(oracle.av_fused(x["attn"], x["v"], case["kernel_size"], case["dilation"]), g("out"), "out")
    else:
        raise AssertionError(kind)
