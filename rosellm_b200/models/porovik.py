"""Porovik as a list of parts.

A decoder-only model whose layers differ in their mixers: causal attention with a distance bias and a
query temperature (no rotation), a generalized delta rule, and a gated linear recurrence, in whatever
order ``config.json`` lists them.  The embedding adds a hashed table of token pairs and a learned position
table; every sublayer has an RMS norm ahead of it and one behind it, with scales kept as offsets from one
(``1 + w``); the feed-forward is dense (tanh-GELU gate) or a mixture of experts (sigmoid scores, the
weight on the expert's input, SiLU gate); a final norm and the embedding table as the head.

Tensor names: ``embed``, ``bigram``, ``pos``, ``final.norm``; layer i: ``l<i>.norm1``, ``l<i>.norm1b``,
``l<i>.norm2``, ``l<i>.norm2b``, ``l<i>.mix.*`` (attention: ``q, k, v, g, o, vmix``; general_delta:
``r, k, v, a, a.b, g, w1, w2, w0, norm, o``; hgrn2: ``q, f, f.b, lower, v, norm, o``) and
``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.router`` with ``l<i>.mlp.e<j>.{gate,up,down}``.  Linear weights
are stored [out, in].
"""
from __future__ import annotations

import math

from ..config.base import register_architecture
from ..config.porovik import PorovikConfig
from ..parts.spec import Concat, LayerSpec, ModelSpec, PartSpec, RunEntry

SLOPE_LOG2_SPAN = 8.0              # attention: slope_h = 2^(-8 (h + 1) / heads)
DELTA_DECAY_SCALE = math.exp(-0.5)  # general_delta: w = exp(-e^(-1/2) sigmoid(.))
DELTA_UNIT_EPS = 1e-6              # general_delta: the unit key's eps


def build_porovik_spec(cfg: PorovikConfig) -> ModelSpec:
    width, eps = cfg.width, cfg.norm_eps

    def norm(name: str) -> PartSpec:
        return PartSpec("rms_norm", dict(hidden_size=width, eps=eps, weight_offset=1.0), {"weight": name})

    layers = []
    value_source_seen = False
    for i, lc in enumerate(cfg.layers):
        p, mx = f"l{i}.", lc.mixer
        if lc.type == "attention":
            mix = None
            if mx.v_mix:
                mix = "mix" if value_source_seen else "source"
                value_source_seen = True
            tensors = {"q_weight": p + "mix.q", "k_weight": p + "mix.k", "v_weight": p + "mix.v",
                       "gate_weight": p + "mix.g", "out_weight": p + "mix.o"}
            if mix is not None:
                tensors["mix_weight"] = p + "mix.vmix"
            mixer = PartSpec(
                "biased_attention",
                dict(hidden_size=width, num_heads=mx.heads, num_kv_heads=mx.kv_heads, key_dim=mx.dim, value_dim=mx.vdim,
                     scale=mx.scale, slope_log2_span=SLOPE_LOG2_SPAN, temp_coef=mx.q_temp_coef, temp_every=mx.q_temp_every,
                     value_mix=mix, gate=True),
                tensors)
        elif lc.type == "general_delta":
            mixer = PartSpec(
                "delta_rule",
                dict(hidden_size=width, num_heads=mx.heads, head_dim=mx.dim, norm_eps=eps, low_rank=mx.decay_rank,
                     decay_scale=DELTA_DECAY_SCALE, unit_eps=DELTA_UNIT_EPS),
                {"r_weight": p + "mix.r", "k_weight": p + "mix.k", "v_weight": p + "mix.v", "a_weight": p + "mix.a",
                 "a_bias": p + "mix.a.b", "g_weight": p + "mix.g", "w1_weight": p + "mix.w1", "w2_weight": p + "mix.w2",
                 "w0": p + "mix.w0", "out_norm": p + "mix.norm", "out_weight": p + "mix.o"})
        else:  # hgrn2
            mixer = PartSpec(
                "gated_recurrence",
                dict(hidden_size=width, num_heads=mx.heads, key_dim=mx.dim, value_dim=mx.vdim, norm_eps=eps),
                {"q_weight": p + "mix.q", "f_weight": p + "mix.f", "f_bias": p + "mix.f.b", "lower": p + "mix.lower",
                 "v_weight": p + "mix.v", "out_norm": p + "mix.norm", "out_weight": p + "mix.o"})
        named = dict(norm_mixer=("norm", norm(p + "norm1")), mixer=("mixer", mixer),
                     norm_mixer_out=("norm", norm(p + "norm1b")))
        if lc.mlp is not None:
            if lc.mlp.kind == "dense":
                ff = PartSpec("gated_mlp", dict(hidden_size=width, inner_size=lc.mlp.ff, gate="gelu_tanh"),
                              {"gate_up_weight": Concat((p + "mlp.gate", p + "mlp.up"), dim=0),
                               "down_weight": p + "mlp.down"})
            else:
                experts = [f"{p}mlp.e{j}." for j in range(lc.mlp.experts)]
                ff = PartSpec(
                    "moe",
                    dict(hidden_size=width, inner_size=lc.mlp.ff, num_experts=lc.mlp.experts, top=lc.mlp.top, gate="silu",
                         score="sigmoid", weight_input=True),
                    {"router_weight": p + "mlp.router",
                     "gate_up_weight": Concat(tuple(e + w for e in experts for w in ("gate", "up")), dim=0),
                     "down_weight": Concat(tuple(e + "down" for e in experts), dim=0)})
            named.update(norm_feed_forward=("norm", norm(p + "norm2")), feed_forward=("feed_forward", ff),
                         norm_feed_forward_out=("norm", norm(p + "norm2b")))
        layers.append(LayerSpec.of(PartSpec("pre_post_norm", dict(feed_forward=lc.mlp is not None)), **named))
    return ModelSpec(
        hidden_size=width,
        vocab_size=cfg.vocab,
        max_positions=cfg.max_positions,
        embedding=PartSpec("token_pair_table",
                           dict(vocab_size=cfg.vocab, hidden_size=width, buckets=cfg.bigram_buckets,
                                mul_prev=cfg.bigram_mul_prev, mul_cur=cfg.bigram_mul_cur),
                           {"weight": "embed", "pair_weight": "bigram"}),
        position=PartSpec("learned_absolute", dict(max_positions=cfg.max_positions, hidden_size=width), {"weight": "pos"}),
        layers=tuple(layers),
        run_order=tuple(RunEntry(i) for i in range(len(cfg.layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("tied_to_embedding", dict(vocab_size=cfg.vocab, hidden_size=width)),
        eos_token_id=cfg.eos_token_id,
    )


register_architecture("Porovik", PorovikConfig, build_porovik_spec, model_types=("porovik",), replace=True)
