"""CPU checks of the boundary: the shared library loads and exports every symbol the header declares
(no compute call is made), the ctypes table covers the header, and the product path refuses to run
without a GPU instead of falling back."""
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "xfold_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(xfold_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg._cabi.load()
    names = header_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/xfold_b200.h but not exported"
    assert set(names) == set(pkg._cabi.SIGNATURES), set(names) ^ set(pkg._cabi.SIGNATURES)
    assert b"sm_100a" in lib.xfold_version()


def test_header_cites_the_reference_interfaces():
    text = open(os.path.join(ROOT, "include", "xfold_b200.h")).read()
    for cite in ("Alpha_Attention.cpp:148-169", "Alpha_Attention.cpp:50-70", "Alpha_Attention.cpp:116-125",
                 "Alpha_Attention.cpp:72-92", "nn/d_pairformer.py:99-171", "no counterpart in the reference"):
        assert cite in text


def test_no_cpu_fallback(pkg, oracle):
    from distributed_xfold_b200 import ops
    from distributed_xfold_b200._cabi import XfoldError
    x = torch.zeros(4, 128, dtype=torch.bfloat16)
    with pytest.raises(XfoldError):
        ops.layernorm(x)
    if not torch.cuda.is_available():
        with pytest.raises(XfoldError):
            pkg._cabi.ctx(0)   # no sm_100 device: the context cannot be created


def test_product_code_does_not_import_the_oracle():
    pkgdir = os.path.join(ROOT, "distributed-xfold_b200")
    for base, _, files in os.walk(pkgdir):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(base, f)).read()
                assert "xfold_oracle" not in src and "load_oracle" not in src, f
                assert "oracle/" not in src, f


def test_sample_sharding_rule(pkg):
    from distributed_xfold_b200.diffusion import shard_samples
    assert [shard_samples(5, 2, r) for r in range(2)] == [slice(0, 3), slice(3, 5)]
    assert [shard_samples(8, 8, r) for r in range(8)] == [slice(i, i + 1) for i in range(8)]


def test_swiglu_weight_packing_roundtrip(pkg):
    from distributed_xfold_b200.ops import pack_swiglu_weight
    w = torch.arange(2 * 256 * 3, dtype=torch.float32).reshape(512, 3)
    p = pack_swiglu_weight(w)
    assert torch.equal(p[:128], w[:128]) and torch.equal(p[128:256], w[256:384])
    assert torch.equal(p[256:384], w[128:256]) and torch.equal(p[384:], w[384:])
