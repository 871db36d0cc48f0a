"""Diagnostic: where the roles of the tensor-core forward spend their cycles.

Needs a build of the library with per-role cycle counters compiled in:

    NATTEN_B200_NVCC_FLAGS="-DNB_SM100_PROFILE" python natten-mlx_b200/build.py --force
    python natten-mlx_b200/probe/role_counters.py [dilation]
    python natten-mlx_b200/build.py --force          # back to the regular build

Runs the forward of the NAT-stage shape (bf16 B=32 56x56 4 heads D=32, kernel 7x7) three times and prints, for
CTA 0 of the last run, the cycles every role spent working and in each of its waits (TMA producer, MMA thread,
softmax warps 0, 1 and 3).  A regular build has no counters and no ``natten_b200_profile_buffer`` symbol.
"""

import ctypes
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

import torch  # noqa: E402

from natten_mlx_b200 import _lib  # noqa: E402
from natten_mlx_b200._core import cuda as backend  # noqa: E402

B = 32
dil = int(sys.argv[1]) if len(sys.argv) > 1 else 1
gen = torch.Generator(device="cuda").manual_seed(0)
q, k, v = (torch.randn((B, 56, 56, 4, 32), generator=gen, device="cuda").to(torch.bfloat16) for _ in range(3))
buf = torch.zeros(((1 << 21) + 64) * 2, device="cuda")        # counters live at u64 slot 2^20 of this buffer
lib = _lib.load()
try:
    setbuf = lib.natten_b200_profile_buffer
except AttributeError:
    raise SystemExit("this build of the library has no cycle counters (see the docstring)")
setbuf.restype, setbuf.argtypes = None, [ctypes.c_void_p]
geom = _lib.make_geom(2, B, 4, 4, 32, _lib.BF16, (56, 56), (7, 7), (1, 1), (dil, dil), [0, 0], 32 ** -0.5)
print(_lib.describe_plan(geom).split(" | ")[0])
for i in range(3):
    if i == 2:
        setbuf(buf.data_ptr())
    backend.fused_forward(q, k, v, (7, 7), (1, 1), (dil, dil), (False, False), None, path="tcgen05")
torch.cuda.synchronize()
setbuf(None)
prof = buf.view(torch.int64)[(1 << 20):(1 << 20) + 48].cpu().tolist()
softmax = ["other", "wait Q", "wait S", "maximum pass", "exponential pass + arrive", "wait O", "epilogue", "total"]
roles = {"producer": (0, ["work", "wait Q stage", "wait K/V stage", "", "", "", "", "total"]),
         "mma thread": (8, ["work", "wait Q", "wait K/V", "wait P", "wait O buffer", "", "", "total"]),
         "softmax warp 0": (16, softmax), "softmax warp 1": (24, softmax), "softmax warp 3": (40, softmax)}
for name, (base, labels) in roles.items():
    print(name + ": " + ", ".join(f"{lab} {c}" for lab, c in zip(labels, prof[base:base + 8]) if lab))
