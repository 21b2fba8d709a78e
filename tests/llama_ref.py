"""A llama forward pass composed from the CPU oracle's ops (test infrastructure): the same node sequence as
llm_build_llama (cactus/llama-model.cpp:4517-4671) with the unified f16 cache, one ubatch at a time."""
import numpy as np

from oracle.binding import Q4_0, Q8_0  # noqa: F401


class OracleLlama:
    def __init__(self, oracle, cfg, arrays, n_cells, acc_mode=0):
        self.o, self.cfg, self.a, self.n_cells, self.acc_mode = oracle, cfg, arrays, n_cells, acc_mode
        kvd = cfg.n_kv_head * cfg.head_dim
        self.kc = [np.zeros((n_cells, cfg.n_kv_head, cfg.head_dim), np.uint16) for _ in range(cfg.n_layer)]
        self.vc = [np.zeros((n_cells, cfg.n_kv_head, cfg.head_dim), np.uint16) for _ in range(cfg.n_layer)]
        self.cell_pos = np.full(n_cells, -1, np.int32)
        self.cell_seq = np.full(n_cells, -1, np.int32)
        del kvd

    def decode(self, tokens, pos, seq, slots):
        o, cfg, a = self.o, self.cfg, self.a
        T, D, H, Hkv = len(tokens), cfg.head_dim, cfg.n_head, cfg.n_kv_head
        pos = np.asarray(pos, np.int32)
        self.cell_pos[slots] = pos
        self.cell_seq[slots] = seq
        mask = o.build_kq_mask(self.n_cells, self.cell_pos, self.cell_seq, pos, np.asarray(seq, np.int32))
        x = o.get_rows(cfg.head_type, a["token_embd.weight"], np.asarray(tokens, np.int32), cfg.d_model)
        for il in range(cfg.n_layer):
            p = f"blk.{il}."
            h = o.rms_norm_mul(x, a[p + "attn_norm.weight"], cfg.eps)
            q, _ = o.mul_mat(cfg.layer_type, a[p + "attn_q.weight"], h)
            k, _ = o.mul_mat(cfg.layer_type, a[p + "attn_k.weight"], h)
            v, _ = o.mul_mat(cfg.layer_type, a[p + "attn_v.weight"], h)
            q = o.rope_norm(q.reshape(T, H, D), pos, cfg.rope_theta)
            k = o.rope_norm(k.reshape(T, Hkv, D), pos, cfg.rope_theta)
            self.kc[il][slots] = o.cpy_f32_f16(k)
            self.vc[il][slots] = o.cpy_f32_f16(v.reshape(T, Hkv, D))
            att = o.flash_attn_ext(q, self.kc[il], self.vc[il], mask, float(D) ** -0.5, n_kv=self.n_cells, acc_mode=self.acc_mode)
            ao, _ = o.mul_mat(cfg.layer_type, a[p + "attn_output.weight"], att.reshape(T, H * D))
            x = o.add(x, ao)
            h = o.rms_norm_mul(x, a[p + "ffn_norm.weight"], cfg.eps)
            g, _ = o.mul_mat(cfg.layer_type, a[p + "ffn_gate.weight"], h)
            u, _ = o.mul_mat(cfg.layer_type, a[p + "ffn_up.weight"], h)
            dn, _ = o.mul_mat(cfg.layer_type, a[p + "ffn_down.weight"], o.silu_mul(g, u))
            x = o.add(x, dn)
        h = o.rms_norm_mul(x, a["output_norm.weight"], cfg.eps)
        logits, _ = o.mul_mat(cfg.head_type, a["output.weight"], h)
        return logits


def tiny_model(oracle, cfg, seed=0):
    """name -> numpy arrays (quantised block streams / f32 norms) for a random model of shape cfg."""
    rng = np.random.default_rng(seed)
    names = {"wq": "attn_q", "wk": "attn_k", "wv": "attn_v", "wo": "attn_output", "gate": "ffn_gate", "up": "ffn_up", "down": "ffn_down"}
    a = {}
    d = cfg.d_model
    a["token_embd.weight"] = oracle.quantize_weights(cfg.head_type, rng.standard_normal((cfg.vocab, d)).astype(np.float32))
    a["output.weight"] = oracle.quantize_weights(cfg.head_type, (rng.standard_normal((cfg.vocab, d)) * 0.05).astype(np.float32))
    a["output_norm.weight"] = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    for il in range(cfg.n_layer):
        for short, K, M in cfg.mul_mat_shapes():
            a[f"blk.{il}.{names[short]}.weight"] = oracle.quantize_weights(cfg.layer_type, (rng.standard_normal((M, K)) * (1.0 / np.sqrt(K))).astype(np.float32))
        a[f"blk.{il}.attn_norm.weight"] = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
        a[f"blk.{il}.ffn_norm.weight"] = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    return a
