"""The ``-DTPB_BOUNDS`` build of the native library: kernels check their store indices against the extents the host
passed and report ``STATUS_BAD_ARG`` instead of touching memory outside them (nothing traps, nothing faults).  The
variant is loaded in a child process through ``TPB_LIB_PATH``; it is built by ``__graft_entry__.build()`` (or here, if
absent or older than the sources, and nvcc is present)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import sys, torch
sys.path.insert(0, %(repo)r)
from tensor_parallel_b200.ops import native as nat
assert nat.LIB.tpb_bounds_checked() == 1, "not the checked build"
dev = torch.device("cuda", 0)
state = nat.device_state(dev)
torch.manual_seed(0)
# correct calls of every epilogue flavour: results right, status word clean
for tokens, features, k, kw in ((8, 1536, 4096, {}), (8, 2752, 4096, {"act": "swiglu16"}), (40, 1000, 512, {"act": "gelu"}), (300, 1000, 520, {}),
                                (8, 1024, 2048, {"force_splits": 3}), (2048, 512, 256, {})):
    x = torch.randn(tokens, k, device=dev, dtype=torch.bfloat16)
    w = torch.randn(features, k, device=dev, dtype=torch.bfloat16) * 0.05
    out = nat.gemm_nt(x, w, **kw)
    ref = x.float() @ w.float().t()
    if kw.get("act") == "swiglu16":
        g = ref.reshape(tokens, -1, 2, 16)
        ref = (torch.nn.functional.silu(g[:, :, 0]) * g[:, :, 1]).reshape(tokens, -1)
    elif kw.get("act") == "gelu":
        ref = torch.nn.functional.gelu(ref)
    torch.cuda.synchronize()
    assert int(state.status[0].item()) == 0, (tokens, features, k, kw)
    err = (out.float() - ref).abs().max().item()
    assert err <= 0.03 * ref.abs().max().item() + 0.05, (tokens, features, k, kw, err)
# a call whose declared output extent is too small for its shape: the stores past it are skipped and reported
for tokens, features, k in ((8, 1024, 512), (300, 512, 256)):
    x = torch.randn(tokens, k, device=dev, dtype=torch.bfloat16)
    w = torch.randn(features, k, device=dev, dtype=torch.bfloat16) * 0.05
    out = torch.full((tokens, features), 7.0, device=dev, dtype=torch.bfloat16)
    declared = (tokens // 2) * features
    nat.gemm_nt(x, w, out=out, out_elems=declared)
    torch.cuda.synchronize()
    assert int(state.status[0].item()) == 3, "an out-of-extent store went unreported"
    state.status.zero_()
    flat = out.reshape(-1)
    assert bool((flat[declared:] == 7.0).all()), "memory past the declared extent was written"
    ref = (x.float() @ w.float().t()).reshape(-1)[:declared]
    assert (flat[:declared].float() - ref).abs().max().item() <= 0.03 * ref.abs().max().item() + 0.05
print("bounds ok")
"""


def test_checked_build_reports_instead_of_writing_out_of_bounds():
    lib = os.path.join(REPO, "tensor_parallel_b200", "lib", "libtpb200_bounds.so")
    csrc = os.path.join(REPO, "tensor_parallel_b200", "csrc")
    newest = max(os.path.getmtime(os.path.join(csrc, f)) for f in os.listdir(csrc))
    if not os.path.exists(lib) or os.path.getmtime(lib) < newest:  # absent, or older than the sources it was built from
        sys.path.insert(0, REPO)
        from tensor_parallel_b200 import build

        build.build(lib_path=lib, extra_flags=["-DTPB_BOUNDS"])
    env = dict(os.environ, TPB_LIB_PATH=lib)
    proc = subprocess.run([sys.executable, "-c", CHILD % {"repo": REPO}], env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0 and "bounds ok" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-4000:]
