"""CPU: the oracle reproduces the golden vectors (the REFERENCE's own outputs, written by
oracle/pin_against_reference.py) from the recorded seeds, on this machine, without the reference tree."""
import pytest
import torch


def range_rel(y, ref):
    return float((y - ref).abs().max() / (ref.max() - ref.min()).clamp_min(1e-30))


def checksum(*ts):
    return float(sum(t.double().abs().sum() for t in ts))


@pytest.mark.parametrize("name", ["trimul/out/n24", "trimul/in/n24", "trimul/out/n40", "trimul/in/n40", "trimul/out/n33",
                                  "trimul/in/n33", "trimul_gloo2/out/n24", "trimul_gloo2/in/n24"])
def test_trimul_golden(oracle, golden, name):
    meta, ref = golden[name]["meta"], golden[name]["out"][0]
    n = meta["n"]
    g = torch.Generator().manual_seed(meta["seed"])
    st = oracle.make_trimul_state(g, "")
    z = torch.randn(n, n, 128, generator=g)
    if name.startswith("trimul_gloo2"):
        mask = torch.rand(n, n, generator=g)
    else:
        r1, r2 = torch.rand(n, n, generator=g), torch.rand(n, n, generator=g)
        mask = {"rand": r1, "ones": torch.ones(n, n), "binary": (r2 > 0.2).float()}[meta["mask"]]
    assert abs(checksum(z, mask, *st.values()) - meta["checksum"]) < 1e-6 * meta["checksum"], "input generation drifted"
    with torch.no_grad():
        out = oracle.triangle_multiplication(st, "", z, mask, meta["outgoing"])
    assert range_rel(out, ref) < 2e-5


def test_pairformer_block_golden(oracle, golden):
    meta = golden["ref/pairformer_block"]["meta"]
    ref_z, ref_s = golden["ref/pairformer_block"]["out"]
    n = meta["n"]
    g = torch.Generator().manual_seed(meta["seed"])
    st = oracle.make_pairformer_block_state(g, "")
    z = torch.randn(n, n, 128, generator=g)
    s = torch.randn(n, 384, generator=g)
    sm = (torch.rand(n, generator=g) > 0.15).float()
    pm = sm[:, None] * sm[None, :]
    assert abs(checksum(z, s, pm, *st.values()) - meta["checksum"]) < 1e-6 * meta["checksum"]
    with torch.no_grad():
        oz, os_ = oracle.pairformer_block(st, "", z, pm, s, sm)
    assert range_rel(oz, ref_z) < 2e-5 and range_rel(os_, ref_s) < 2e-5


def test_diffusion_transformer_golden(oracle, golden):
    meta, ref = golden["ref/diffusion_transformer"]["meta"], golden["ref/diffusion_transformer"]["out"][0]
    g = torch.Generator().manual_seed(meta["seed"])
    st = oracle.make_diffusion_transformer_state(g, "", meta["c_act"], meta["c_cond"], meta["c_pair"], meta["heads"],
                                                 meta["blocks"], meta["super"])
    n = meta["n"]
    act = torch.randn(2, n, meta["c_act"], generator=g)
    cond = torch.randn(n, meta["c_cond"], generator=g)
    pc = torch.randn(n, n, meta["c_pair"], generator=g)
    mask = (torch.rand(n, generator=g) > 0.2)
    with torch.no_grad():
        out = oracle.diffusion_transformer(st, "", act, mask.float(), cond, pc, meta["heads"], meta["blocks"], meta["super"])
    assert range_rel(out, ref) < 2e-5


def test_sharded_emulation_equals_unsharded(oracle):
    """The oracle's P-rank emulation (TriMul on the full pair, attention on row / column shards)."""
    g = torch.Generator().manual_seed(3)
    st = oracle.make_pairformer_block_state(g, "")
    z, s, pm, sm = oracle.make_inputs(4, 18, pad_frac=0.1)
    with torch.no_grad():
        a = oracle.pairformer_block(st, "", z, pm, s, sm)
        b = oracle.pairformer_block_sharded(st, "", z, pm, s, sm, 4)
    assert oracle.rel_frobenius(b[0], a[0]) < 1e-5 and oracle.rel_frobenius(b[1], a[1]) < 1e-5


def test_row_chunked_attention_equals_full(oracle):
    g = torch.Generator().manual_seed(5)
    st = oracle.make_grid_attention_state(g, "")
    z, _, pm, _ = oracle.make_inputs(6, 20, pad_frac=0.1)
    with torch.no_grad():
        a = oracle.grid_self_attention(st, "", z, pm, z, False)
        b = oracle.grid_self_attention(st, "", z, pm, z, False, row_chunk=7)
    assert torch.allclose(a, b, atol=1e-5)


def cross_attention_inputs(meta):
    """The inputs the pin script drew for ``spec/cross_attention`` (parameters in the spec class's declaration order)."""
    B, S, K, c, H = meta["B"], meta["S"], meta["K"], meta["c"], meta["H"]
    D = c // H
    g = torch.Generator().manual_seed(meta["seed"])
    ws = {}
    for name, shape in (("query_w", (c, H, D)), ("query_b", (1, H, D)), ("key_w", (c, H, D)), ("value_w", (c, H, D)),
                        ("gating_w", (c, H, D))):
        ws[name] = torch.randn(shape, generator=g) / 8
    qd = torch.randn(B, S, c, generator=g)
    md = torch.randn(B, K, c, generator=g)
    bb = torch.randn(B, H, S, K, generator=g)
    bb = bb + 1e9 * ((torch.rand(B, 1, 1, K, generator=g) > 0.1).float() - 1)
    return qd, md, bb, ws


def test_cross_attention_golden(oracle, golden):
    """The reference's CrossAttention spec class (kernel_test/batch_diffusion_cross_attention.py:23-87)."""
    meta, ref = golden["spec/cross_attention"]["meta"], golden["spec/cross_attention"]["out"][0]
    qd, md, bb, ws = cross_attention_inputs(meta)
    assert abs(checksum(qd, md, bb, *ws.values()) - meta["checksum"]) < 1e-6 * meta["checksum"], "input generation drifted"
    out = oracle.cross_attention(qd, md, bb, ws["query_w"], ws["query_b"], ws["key_w"], ws["value_w"], ws["gating_w"])
    assert range_rel(out, ref) < 2e-5
