"""Host reference of the decoder-stack composition, built from the CPU oracle's pinned operators with BF16 rounding
at every activation boundary.  PARITY UNPINNED with respect to the reference: no rust-ascend test fixes a Llama
forward value (its Llama lives in the external RUDA crates); this states the standard pre-norm block."""
import numpy as np

from rust_ascend_b200.decoder import LlamaConfig, WeightSource, rope_tables, shard_plan
from rust_ascend_b200.runtime import bf16_bits_to_f32


def full_weights(cfg: LlamaConfig, seed: int):
    src = WeightSource(seed, exact=True)
    f = lambda *a, **k: bf16_bits_to_f32(src.matrix(*a, **k))
    h, d = cfg.hidden, cfg.head_dim
    w = {"embedding": f("embedding", 0, cfg.vocab, h), "lm_head": f("lm_head", 0, cfg.vocab, h), "layers": []}
    for li in range(cfg.layers):
        w["layers"].append({"wq": f("wq", li, cfg.heads * d, h), "wk": f("wk", li, cfg.kv_heads * d, h), "wv": f("wv", li, cfg.kv_heads * d, h),
                            "wo": f("wo", li, h, cfg.heads * d), "wg": f("wg", li, cfg.ffn, h), "wu": f("wu", li, cfg.ffn, h),
                            "wd": f("wd", li, h, cfg.ffn)})
    return w


def forward(orc, cfg: LlamaConfig, weights, tokens, rank=0, world=1, all_reduce=None):
    """Logits [T, vocab/world].  With world > 1 the projections use this rank's shards and `all_reduce(array)` sums
    the row-parallel partial results over ranks."""
    b, s = tokens.shape
    t, d = b * s, cfg.head_dim
    p = shard_plan(cfg, rank, world)
    hq, hkv = p["q_heads"], p["kv_heads"]
    ones = np.ones(cfg.hidden, np.float32)
    cos, sin = rope_tables(s, d, cfg.theta)
    R = orc.bf16
    rs = lambda a, r: a[r[0]:r[1]]
    x = weights["embedding"][tokens.reshape(-1)]
    for lw in weights["layers"]:
        h = R(orc.rms_norm(x, ones, cfg.eps)[0])
        q = R(orc.linear(h, rs(lw["wq"], p["q_rows"]))).reshape(b, s, hq, d).transpose(0, 2, 1, 3)
        k = R(orc.linear(h, rs(lw["wk"], p["kv_rows"]))).reshape(b, s, hkv, d).transpose(0, 2, 1, 3)
        v = R(orc.linear(h, rs(lw["wv"], p["kv_rows"]))).reshape(b, s, hkv, d).transpose(0, 2, 1, 3)
        q = R(orc.rotary(q, np.broadcast_to(cos, (b, hq, s, d // 2)), np.broadcast_to(sin, (b, hq, s, d // 2)), "split_half"))
        k = R(orc.rotary(k, np.broadcast_to(cos, (b, hkv, s, d // 2)), np.broadcast_to(sin, (b, hkv, s, d // 2)), "split_half"))
        a = orc.attention(q, k, v, 1.0 / np.sqrt(d), causal=True, out_bf16=True).transpose(0, 2, 1, 3).reshape(t, hq * d)
        o = R(orc.linear(a, lw["wo"][:, p["o_cols"][0]:p["o_cols"][1]]))
        if all_reduce is not None:
            o = R(all_reduce(o))
        x = R(x + o)
        h = R(orc.rms_norm(x, ones, cfg.eps)[0])
        g = R(orc.linear(h, rs(lw["wg"], p["ffn_rows"]), w_up=rs(lw["wu"], p["ffn_rows"])))
        dn = R(orc.linear(g, lw["wd"][:, p["down_cols"][0]:p["down_cols"][1]]))
        if all_reduce is not None:
            dn = R(all_reduce(dn))
        x = R(x + dn)
    h = R(orc.rms_norm(x, ones, cfg.eps)[0])
    return R(orc.linear(h, rs(weights["lm_head"], p["vocab_rows"])))
