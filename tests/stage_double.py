"""CPU stand-in for the stage backend of ``row_sharded.pairformer_block`` built on the oracle
(test infrastructure): same interface and tensor layouts as ``CudaStages``, fp32 torch arithmetic.
It lets the gloo tests check the sharding algebra of the multi-rank block without a GPU."""
import torch
import torch.nn.functional as F


class Weights:
    def __init__(self, state, prefix, with_single=True):
        self.state, self.prefix, self.with_single = state, prefix, with_single
        self.tri_out = (state, prefix + "triangle_multiplication_outgoing.")
        self.tri_in = (state, prefix + "triangle_multiplication_incoming.")
        self.att_start = (state, prefix + "pair_attention1.")
        self.att_end = (state, prefix + "pair_attention2.")
        self.pair_transition = (state, prefix + "pair_transition.")


def _pad8(n):
    return (n + 7) // 8 * 8


class OracleStages:
    def __init__(self, oracle):
        self.O = oracle

    def trimul_project(self, z, mask_shard, w):
        st, p = w
        x = self.O.layer_norm(z, st.get(p + "left_norm_input.weight"), st.get(p + "left_norm_input.bias"))
        pr = F.linear(x, st[p + "projection.weight"])
        if mask_shard is not None:
            pr = pr * mask_shard[..., None]
        pr = pr * torch.sigmoid(F.linear(x, st[p + "gate.weight"]))
        a = pr[..., 0::2].permute(0, 2, 1).contiguous()   # [R, c, N]
        b = pr[..., 1::2].permute(0, 2, 1).contiguous()
        return a, b, F.linear(x, st[p + "gating_linear.weight"])

    def trimul_contract(self, a, b_full, n):
        return torch.einsum("ick,jck->icj", a[..., :n], b_full[..., :n])

    def trimul_contract_planes(self, a, b, n):
        return torch.einsum("cik,cjk->cij", a[..., :n], b[..., :n])

    def trimul_output(self, o, g, z, w):
        st, p = w
        y = self.O.layer_norm(o.permute(0, 2, 1), st.get(p + "center_norm.weight"), st.get(p + "center_norm.bias"))
        z += F.linear(y, st[p + "output_projection.weight"]) * torch.sigmoid(g)

    def triattn_bias(self, z, w, rows_are_keys):
        st, p = w
        x = self.O.layer_norm(z, st.get(p + "act_norm.weight"), st.get(p + "act_norm.bias"))
        nb = F.linear(x, st[p + "pair_bias_projection.weight"])     # [R, N, 4]
        if rows_are_keys:
            return x, nb.permute(2, 1, 0).contiguous()              # [4, N(query), R(key)]
        out = torch.zeros(4, z.shape[0], _pad8(z.shape[1]))
        out[..., : z.shape[1]] = nb.permute(2, 0, 1)                # [4, R(query), N(key)]
        return x, out

    def triattn_core(self, x, bias, mask_shard, w, z):
        st, p = w
        r, n, c = x.shape
        h, d = 4, c // 4
        q = F.linear(x, st[p + "q_projection.weight"]).reshape(r, n, h, d).permute(0, 2, 1, 3) * d ** -0.5
        k = F.linear(x, st[p + "k_projection.weight"]).reshape(r, n, h, d).permute(0, 2, 1, 3)
        v = F.linear(x, st[p + "v_projection.weight"]).reshape(r, n, h, d).permute(0, 2, 1, 3)
        logits = q @ k.transpose(-1, -2) + bias[:, :n, :n][None]
        if mask_shard is not None:
            logits = logits + 1e9 * (mask_shard[:, None, None, :] - 1)
        o = (torch.softmax(logits, -1) @ v).permute(0, 2, 1, 3).reshape(r, n, c)
        o = o * torch.sigmoid(F.linear(x, st[p + "gating_query.weight"]))
        z += F.linear(o, st[p + "output_projection.weight"])

    def transition(self, z, w):
        st, p = w
        z += self.O.transition(st, p, z)

    def pair_logits(self, z, w):
        st, p = w.state, w.prefix
        x = self.O.layer_norm(z, st.get(p + "single_pair_logits_norm.weight"), st.get(p + "single_pair_logits_norm.bias"))
        out = torch.zeros(16, z.shape[0], _pad8(z.shape[1]))
        out[..., : z.shape[1]] = F.linear(x, st[p + "single_pair_logits_projection.weight"]).permute(2, 0, 1)
        return out                                                  # [16, R(query), pad8(N)(key)]

    def single_update(self, s, pl, seq_mask, w):
        st, p = w.state, w.prefix
        n = s.shape[0]
        s += self.O.self_attention(st, p + "single_attention_.", s, seq_mask, pl[:, :n, :n], None, 16)
        s += self.O.transition(st, p + "single_transition.", s)
