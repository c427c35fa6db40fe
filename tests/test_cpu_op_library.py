"""CPU: the Meta kernels registered for ``torch.ops._alpha_attention.*`` give the padded shapes of the reference's own
shape-only kernels (xsmm_kernels/prototypes/register_fake_kernels.py:12-125): sequence axes rounded up to 64,
TriangleMultiplication's two token axes to 32."""
import torch


def test_meta_shapes(pkg):
    from distributed_xfold_b200 import op_library
    op_library.register()
    op_library.register()   # idempotent
    ops = torch.ops._alpha_attention
    m = lambda *s: torch.empty(*s, device="meta", dtype=torch.bfloat16)
    f = lambda *s: torch.empty(*s, device="meta")
    assert tuple(ops.traingle_multiplication_forward(m(70, 70, 128), f(70, 70, 1), 0, m(128), m(128), m(256, 128), m(256, 128),
                                                     m(128), m(128), m(128, 128), m(128, 128)).shape) == (96, 96, 128)
    assert tuple(ops.grid_self_attn_forward(m(5, 70, 128), f(5, 1, 1, 70), f(4, 70, 70), m(128, 4, 32), m(128, 4, 32),
                                            m(128, 4, 32), m(128, 4, 32), m(4, 32, 128), 32, 32).shape) == (5, 128, 128)
    assert tuple(ops.batch_diffusion_self_attention_forward(m(2, 64, 768), f(1, 1, 1, 64), f(16, 64, 64), m(768, 16, 48),
                                                            f(1, 16, 48), m(768, 16, 48), m(768, 16, 48), m(768, 16, 48), 48,
                                                            48).shape) == (2, 64, 16, 48)
    assert tuple(ops.batch_diffusion_cross_attention_forward(m(9, 32, 128), m(9, 128, 128), f(9, 4, 32, 128), m(128, 4, 32),
                                                             f(1, 4, 32), m(128, 4, 32), m(128, 4, 32), m(128, 4, 32), 32,
                                                             32).shape) == (9, 64, 4, 32)
    assert tuple(ops.transition_forward(m(3, 7, 128), m(128, 1024), f(512, 128), m(128), m(128)).shape) == (3, 7, 128)


_WRAPPER_SCRIPT = r"""
import sys, torch
repo, ref_src = sys.argv[1], sys.argv[2]
sys.path.insert(0, repo)
import __graft_entry__ as ge
ge.load_package()
sys.path.insert(0, repo + "/oracle")
import ref_standins
ref_standins.install(ref_src)                                # stand-ins for the absent third-party packages
import distributed_xfold.xsmm_kernels.prototypes as P        # the reference's own wrappers and shape-only kernels
from distributed_xfold_b200 import op_library
op_library.register()                                        # must coexist with schemas somebody else defined
from distributed_xfold.xsmm_kernels.prototypes.TriangleMultiplication import TriangleMultiplicationFunction
m = lambda *s: torch.empty(*s, device="meta", dtype=torch.bfloat16)
f = lambda *s: torch.empty(*s, device="meta")
for eq in ("ikc,jkc->ijc", "kjc,kic->ijc"):
    out = TriangleMultiplicationFunction.apply(m(70, 70, 128), f(70, 70, 1), eq, m(128), m(128), m(256, 128), m(256, 128),
                                               m(128), m(128), m(128, 128), m(128, 128))
    assert tuple(out.shape) == (70, 70, 128), out.shape     # padded to 96 by the op, narrowed by the wrapper
print("wrappers ok")
"""


def test_reference_wrappers_run_on_the_registered_ops(pkg, tmp_path):
    """With a checkout of the reference beside this repository, its own wrapper
    (xsmm_kernels/prototypes/TriangleMultiplication.py:19-59: call the op, narrow the padded result) runs unchanged on
    the operators this package registers.  In a child process: the stand-in modules must not leak into other tests."""
    import os
    import subprocess
    import sys
    import pytest
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref_src = os.path.join(os.path.dirname(repo), "reference", "src")
    if not os.path.isdir(os.path.join(ref_src, "distributed_xfold")):
        pytest.skip("no checkout of the reference beside the repository")
    script = tmp_path / "wrappers.py"
    script.write_text(_WRAPPER_SCRIPT)
    r = subprocess.run([sys.executable, str(script), repo, ref_src], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "wrappers ok" in r.stdout, r.stdout + r.stderr
