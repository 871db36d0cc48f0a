"""Generate the golden fixtures in this folder from the reference's own code.

Run where the reference sources are present:

    python tests/golden/make_golden.py /path/to/reference

Files written next to this script:

* ``window_tables.npz``  - integer window starts / ends / bias starts produced
  by the reference's ``utils/window.py`` (pure numpy, loaded as is) over a grid
  of (length, kernel, dilation), plus the dilation-group start formula of
  ``extras/allin1/reference_impl.py``.
* ``pure_cases.npz`` + ``pure_cases.json`` - results of the reference's
  ``_core/pure.py``, ``functional.py``, ``merge.py`` and ``extras/allin1`` on
  seeded inputs.  These modules need the MLX array library, which does not
  install on Linux; ``mlx_stand_in.py`` supplies those array calls with torch
  on the CPU so that the reference's own Python runs unmodified.

Inputs are not stored: each case records its numpy seed and shapes, and
``make_inputs`` below rebuilds them (the tests import it).
"""

from __future__ import annotations

import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

WINDOW_LENGTHS = list(range(1, 41)) + [56, 64, 96, 97, 128]
WINDOW_KERNELS = [1, 2, 3, 4, 5, 6, 7, 8, 9, 13]
WINDOW_DILATIONS = [1, 2, 3, 4, 5, 8]


def window_grid():
    for length in WINDOW_LENGTHS:
        for k in WINDOW_KERNELS:
            for d in WINDOW_DILATIONS:
                if k * d <= length:
                    yield length, k, d


# ---------------------------------------------------------------------------
# seeded float cases
# ---------------------------------------------------------------------------
# kind: fused | qk | av | lse_extra | varlen | merge | qk_rpb | av_fused
def _c(kind, shape, k, s=1, d=1, c=False, **kw):
    return dict(kind=kind, shape=list(shape), kernel_size=k, stride=s, dilation=d, is_causal=c, **kw)


CASES = [
    # the parity configuration: na1d fp32 B=2 L=64 H=4 D=32 K=7, sum-of-outputs loss
    _c("fused", (2, 64, 4, 32), 7, ones_cotangent=True),
    _c("fused", (2, 19, 2, 8), 5, 1, 1, True),
    _c("fused", (1, 23, 3, 4), 3, 2, 3, False),
    _c("fused", (1, 24, 2, 8), 9, 2, 2, True),
    _c("fused", (1, 12, 2, 4), 4, 1, 1, False),            # even kernel
    _c("fused", (1, 6, 2, 4), 6, 1, 1, False),             # even kernel == extent (start -1)
    _c("fused", (1, 9, 2, 4), 9, 1, 1, False),             # kernel covers the extent
    _c("fused", (2, 9, 11, 2, 8), (3, 5), 1, (2, 1), False),
    _c("fused", (1, 12, 10, 2, 4), (5, 3), (2, 1), (1, 3), (True, False)),
    _c("fused", (1, 14, 14, 2, 16), 7, 1, 2, False),
    _c("fused", (1, 8, 8, 4, 8), (3, 3), 1, 1, False, heads_kv=2),
    _c("fused", (1, 5, 7, 8, 2, 4), (3, 3, 5), 1, 1, (True, False, False)),
    _c("fused", (1, 6, 9, 7, 2, 4), (3, 3, 3), (1, 2, 1), (2, 3, 1), False),
    _c("qk", (2, 21, 2, 8), 5, 2, 2, True),
    _c("qk", (1, 10, 12, 2, 4), (3, 5), (1, 2), (3, 2), (False, True)),
    _c("qk", (1, 4, 6, 9, 2, 4), (3, 3, 3), 1, (1, 2, 3), (True, False, False)),
    _c("av", (2, 21, 2, 8), 5, 2, 2, True),
    _c("av", (1, 10, 12, 2, 4), (3, 5), (1, 2), (3, 2), (False, True)),
    _c("av", (1, 4, 6, 9, 2, 4), (3, 3, 3), 1, (1, 2, 3), (True, False, False)),
    _c("lse_extra", (2, 17, 4, 8), 5, 1, 2, False, heads_kv=2, n_extra=3),
    _c("lse_extra", (1, 9, 10, 4, 8), (3, 5), 1, 1, (True, False), heads_kv=1, n_extra=5),
    _c("lse_extra", (1, 4, 6, 5, 2, 4), 3, 1, 1, False, heads_kv=2, n_extra=2),
    _c("lse_extra", (1, 12, 2, 8), 5, 2, 1, False, heads_kv=2, n_extra=0),   # return_lse only, strided
    _c("lse_extra", (1, 5, 6, 2, 8), (5, 6), 1, 1, False, heads_kv=2, n_extra=4),  # dense-attention route
    _c("varlen", (3, 20, 2, 8), 5, 1, 2, False, sizes=[[20], [10], [13]]),
    _c("varlen", (3, 10, 12, 2, 4), (3, 5), 1, (2, 1), False, sizes=[[10, 12], [6, 5], [7, 9]]),
    _c("varlen", (2, 5, 6, 7, 2, 4), 3, 1, 1, False, sizes=[[5, 6, 7], [3, 4, 5]]),
    _c("merge", (2, 6, 5, 3, 8), 0, n_parts=3),
    _c("qk_rpb", (4, 216, 2, 12), 5, 1, 1), _c("qk_rpb", (2, 50, 2, 12), 5, 1, 2),
    _c("qk_rpb", (2, 50, 2, 12), 3, 1, 4), _c("qk_rpb", (1, 64, 2, 12), 7, 1, 8),
    _c("qk_rpb", (1, 40, 3, 6), 5, 1, 1, no_rpb=True),
    _c("qk_rpb", (2, 9, 14, 2, 12), 3, 1, 1), _c("qk_rpb", (1, 12, 23, 2, 12), 5, 1, 2),
    _c("qk_rpb", (1, 16, 15, 2, 4), 7, 1, 2),
    _c("av_fused", (2, 50, 2, 12), 5, 1, 2), _c("av_fused", (1, 12, 23, 2, 12), 5, 1, 2),
]


def _tup(x, rank):
    return tuple(x) if isinstance(x, (list, tuple)) else (x,) * rank


def make_inputs(idx, case):
    """Seeded float32 inputs of a case as a dict of numpy arrays."""
    rng = np.random.default_rng(9000 + idx)
    shape = tuple(case["shape"])
    rank = len(shape) - 3
    kv_shape = shape[:-2] + (case.get("heads_kv", shape[-2]), shape[-1])
    n = lambda s, scale=1.0: (rng.standard_normal(s) * scale).astype(np.float32)
    kind = case["kind"]
    ks = _tup(case["kernel_size"], rank)
    st = _tup(case["stride"], rank)
    outs = tuple(-(-shape[1 + a] // st[a]) for a in range(rank))
    kvol = int(np.prod(ks)) if kind != "merge" else 0
    d = {}
    if kind in ("fused", "varlen"):
        d.update(q=n(shape), k=n(kv_shape), v=n(kv_shape))
        d["cot"] = np.ones((shape[0],) + outs + shape[-2:], np.float32) if case.get("ones_cotangent") \
            else n((shape[0],) + outs + shape[-2:])
    elif kind == "qk":
        d.update(q=n(shape), k=n(shape), cot=n((shape[0],) + outs + (shape[-2], kvol)))
    elif kind == "av":
        d.update(attn=n((shape[0],) + outs + (shape[-2], kvol)), v=n(shape),
                 cot=n((shape[0],) + outs + shape[-2:]))
    elif kind == "lse_extra":
        d.update(q=n(shape), k=n(kv_shape), v=n(kv_shape))
        ne = case["n_extra"]
        if ne:
            d.update(ak=n((shape[0], ne, kv_shape[-2], shape[-1])), av=n((shape[0], ne, kv_shape[-2], shape[-1])))
        d.update(cot=n((shape[0],) + outs + shape[-2:]), cot_lse=n((shape[0],) + outs + (shape[-2],)))
    elif kind == "merge":
        for i in range(case["n_parts"]):
            d[f"o{i}"] = n(shape)
            d[f"l{i}"] = n(shape[:-1], 2.0)
    elif kind == "qk_rpb":
        k1 = case["kernel_size"]
        d.update(q=n(shape), k=n(shape))
        if not case.get("no_rpb"):
            d["rpb"] = n((shape[-2],) + (2 * k1 - 1,) * rank, 0.02)
    elif kind == "av_fused":
        k1 = case["kernel_size"]
        d.update(attn=n(shape[:-1] + (k1 ** rank,)), v=n(shape))
    return d


def main(ref_root):
    sys.path.insert(0, HERE)
    import torch
    import mlx_stand_in
    ns = mlx_stand_in.load_reference(os.path.join(ref_root, "src"))
    win = ns.window

    # ---- integer tables -----------------------------------------------------
    starts, ends, pbs, grouped, offsets = [], [], [], [], []
    for length, k, d in window_grid():
        pos = np.arange(length)
        s, e = win.compute_window_start_end(pos, length, k, d)
        p = win.compute_pb_start(pos, length, k, d)
        g = [ns.allin1_ref.get_window_start(int(i), length, k, k // 2, d) for i in pos]
        offsets.append(len(starts))
        starts += s.tolist(); ends += e.tolist(); pbs += p.tolist(); grouped += g
    np.savez_compressed(
        os.path.join(HERE, "window_tables.npz"),
        grid=np.array(list(window_grid()), dtype=np.int16),
        offsets=np.array(offsets, dtype=np.int32),
        starts=np.array(starts, dtype=np.int16), ends=np.array(ends, dtype=np.int16),
        pb_starts=np.array(pbs, dtype=np.int16), grouped_starts=np.array(grouped, dtype=np.int16))

    # per-axis index/valid tables of the pure backend (causal and not, strided)
    axis_cases, axis_idx, axis_ok = [], [], []
    for length, k, d, stride, causal in [(17, 5, 2, 1, False), (17, 5, 2, 2, True), (9, 9, 1, 1, False),
                                         (6, 6, 1, 1, False), (31, 7, 4, 3, False), (12, 4, 3, 1, True)]:
        qp = ns.pure._query_positions(length, stride)
        idx, ok = ns.pure._compute_axis_indices(qp, length, k, d, causal)
        axis_cases.append([length, k, d, stride, int(causal), idx.shape[0]])
        axis_idx.append(idx.reshape(-1)); axis_ok.append(ok.reshape(-1))
    lin2, ok2 = ns.pure._compute_neighbor_indices_2d(7, 9, (3, 5), (2, 1), (True, False))
    lin3, ok3 = ns.pure._compute_neighbor_indices_3d(4, 5, 6, (3, 3, 5), (1, 1, 1), (False, True, False))
    np.savez_compressed(
        os.path.join(HERE, "index_tables.npz"),
        axis_cases=np.array(axis_cases, dtype=np.int32),
        axis_idx=np.concatenate(axis_idx).astype(np.int32), axis_ok=np.concatenate(axis_ok),
        lin2=lin2.numpy(), ok2=ok2.numpy(), lin3=lin3.numpy(), ok3=ok3.numpy())

    # ---- float cases --------------------------------------------------------
    F = ns.functional
    fused = {1: F.na1d, 2: F.na2d, 3: F.na3d}
    qk = {1: F.na1d_qk, 2: F.na2d_qk, 3: F.na3d_qk}
    av = {1: F.na1d_av, 2: F.na2d_av, 3: F.na3d_av}
    varlen = {1: F.na1d_varlen, 2: F.na2d_varlen, 3: F.na3d_varlen}
    P = ns.pure
    bwd = {1: P.na1d_backward, 2: P.na2d_backward, 3: P.na3d_backward}
    qk_bwd = {1: P.na1d_qk_backward, 2: P.na2d_qk_backward, 3: P.na3d_qk_backward}
    av_bwd = {1: P.na1d_av_backward, 2: P.na2d_av_backward, 3: P.na3d_av_backward}
    vl_bwd = {1: P.na1d_varlen_backward, 2: P.na2d_varlen_backward, 3: P.na3d_varlen_backward}

    out = {}
    for i, case in enumerate(CASES):
        x = {k_: torch.from_numpy(v_) for k_, v_ in make_inputs(i, case).items()}
        rank = len(case["shape"]) - 3
        ks, st = _tup(case["kernel_size"], rank), _tup(case["stride"], rank)
        dl, ca = _tup(case["dilation"], rank), _tup(case["is_causal"], rank)
        kind = case["kind"]
        res = {}
        if kind == "fused":
            res["out"] = fused[rank](x["q"], x["k"], x["v"], kernel_size=ks, stride=st, dilation=dl, is_causal=ca)
            rep = x["q"].shape[-2] // x["k"].shape[-2]
            dense = all(k_ >= e_ for k_, e_ in zip(ks, case["shape"][1:1 + rank])) \
                and all(s_ == 1 for s_ in st) and not any(ca)
            if rep == 1 and not dense:
                res["dq"], res["dk"], res["dv"] = bwd[rank](x["q"], x["k"], x["v"], x["cot"], ks, st, dl, ca, None)
            else:  # GQA or the dense route: gradient of the public functional itself
                def loss(q_, k_, v_):
                    return (fused[rank](q_, k_, v_, kernel_size=ks, stride=st, dilation=dl, is_causal=ca) * x["cot"]).sum()
                leaves = [t.clone().requires_grad_(True) for t in (x["q"], x["k"], x["v"])]
                res["dq"], res["dk"], res["dv"] = torch.autograd.grad(loss(*leaves), leaves)
        elif kind == "qk":
            res["out"] = qk[rank](x["q"], x["k"], ks, dl, stride=st, is_causal=ca)
            res["dq"], res["dk"] = qk_bwd[rank](x["q"], x["k"], x["cot"], ks, st, dl, ca, None)
        elif kind == "av":
            res["out"] = av[rank](x["attn"], x["v"], ks, dl, stride=st, is_causal=ca)
            res["dattn"], res["dv"] = av_bwd[rank](x["attn"], x["v"], x["cot"], ks, st, dl, ca)
        elif kind == "lse_extra":
            kw = {}
            if "ak" in x:
                kw = dict(additional_keys=x["ak"], additional_values=x["av"])
            names = ["q", "k", "v"] + (["ak", "av"] if "ak" in x else [])
            leaves = [x[n_].clone().requires_grad_(True) for n_ in names]
            kw2 = dict(kw)
            if "ak" in x:
                kw2 = dict(additional_keys=leaves[3], additional_values=leaves[4])
            o, l = fused[rank](leaves[0], leaves[1], leaves[2], kernel_size=ks, stride=st, dilation=dl,
                               is_causal=ca, return_lse=True, **kw2)
            res["out"], res["lse"] = o.detach(), l.detach()
            g = torch.autograd.grad((o * x["cot"]).sum() + (l * x["cot_lse"]).sum(), leaves)
            for n_, g_ in zip(names, g):
                res["d" + n_] = g_
        elif kind == "varlen":
            sizes = torch.tensor(case["sizes"], dtype=torch.int32)
            if rank == 1:
                sizes = sizes.reshape(-1)
            res["out"] = varlen[rank](x["q"], x["k"], x["v"], sizes, ks, dl)
            res["dq"], res["dk"], res["dv"] = vl_bwd[rank](x["q"], x["k"], x["v"], x["cot"], sizes, ks, dl, None)
        elif kind == "merge":
            n_parts = case["n_parts"]
            res["out"], res["lse"] = ns.merge.merge_attentions([x[f"o{j}"] for j in range(n_parts)],
                                                               [x[f"l{j}"] for j in range(n_parts)])
        elif kind == "qk_rpb":
            f = ns.allin1.na1d_qk_rpb if rank == 1 else ns.allin1.na2d_qk_rpb
            res["out"] = f(x["q"], x["k"], x.get("rpb"), case["kernel_size"], case["dilation"], scale=0.288)
        elif kind == "av_fused":
            f = ns.allin1.na1d_av_fused if rank == 1 else ns.allin1.na2d_av_fused
            res["out"] = f(x["attn"], x["v"], case["kernel_size"], case["dilation"])
        for name, t in res.items():
            out[f"c{i}_{name}"] = t.detach().numpy().astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "pure_cases.npz"), **out)
    with open(os.path.join(HERE, "pure_cases.json"), "w") as fh:
        json.dump(CASES, fh, indent=0)
    print("wrote", len(CASES), "cases;",
          {f: os.path.getsize(os.path.join(HERE, f)) for f in ("window_tables.npz", "index_tables.npz", "pure_cases.npz")})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
