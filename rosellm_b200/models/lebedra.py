"""Lebedra as a list of parts.

A decoder-only model whose sublayers read the residual stream itself and are RMS-normalised
on their way back into it (``x += m * norm(sublayer(x))``): a latent-attention mixer with
rotated query/key parts and a softmax sink, then a gated feed-forward (dense with a ReLU gate,
or a mixture of experts with a clamped swish gate, group-limited choice and a choice
correction; a layer may have none), then a per-layer token-gated input from a second
embedding table.  No position table; a final RMS norm and an untied head.

Tensor names: ``embed``, ``side.embed``, ``final.norm``, ``head``; layer i: ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.{q,dkv,dkv.norm,uk,uv,sink,o}``, ``l<i>.mlp.{gate,up,down}`` or
``l<i>.mlp.{router,correction}`` with ``l<i>.mlp.e<j>.{gate,up,down}``, and
``l<i>.side.{gate,proj,norm}``.  Linear weights are stored [out, in].
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.lebedra import LebedraConfig
from ..parts.spec import Concat, LayerSpec, ModelSpec, PartSpec, RunEntry

SWISH_ALPHA = 1.702  # the experts' gate: g * sigmoid(1.702 g)


def build_lebedra_spec(cfg: LebedraConfig) -> ModelSpec:
    width, eps = cfg.width, cfg.norm_eps
    n_layers = len(cfg.layers)

    def norm(name: str) -> PartSpec:
        return PartSpec("rms_norm", dict(hidden_size=width, eps=eps), {"weight": name})

    layers = []
    for i, lc in enumerate(cfg.layers):
        p, mx = f"l{i}.", lc.mixer
        named = dict(
            mixer=("mixer", PartSpec(
                "latent_attention",
                dict(hidden_size=width, num_heads=mx.heads, plain_dim=mx.dim, rot_dim=mx.rot_dim, value_dim=mx.vdim,
                     kv_rank=mx.kv_rank, scale=mx.scale, rot_dims=mx.rot_dims, rot_base=mx.rot_base, norm_eps=eps,
                     sink=True),
                {"q_weight": p + "mix.q", "dkv_weight": p + "mix.dkv", "dkv_norm": p + "mix.dkv.norm",
                 "uk_weight": p + "mix.uk", "uv_weight": p + "mix.uv", "o_weight": p + "mix.o",
                 "sink": p + "mix.sink"})),
            norm_mixer=("norm", norm(p + "norm1")),
        )
        if lc.mlp is not None and lc.mlp.kind == "dense":
            named["feed_forward"] = ("feed_forward", PartSpec(
                "gated_mlp", dict(hidden_size=width, inner_size=lc.mlp.ff, gate="relu"),
                {"gate_up_weight": Concat((p + "mlp.gate", p + "mlp.up"), dim=0), "down_weight": p + "mlp.down"}))
        elif lc.mlp is not None:
            m = lc.mlp
            experts = [f"{p}mlp.e{j}." for j in range(m.experts)]
            named["feed_forward"] = ("feed_forward", PartSpec(
                "moe",
                dict(hidden_size=width, inner_size=m.ff, num_experts=m.experts, top=m.top, group_count=m.group_count,
                     group_keep=m.group_keep, gate="clamped_swish", alpha=SWISH_ALPHA, limit=m.limit, correction=True),
                {"router_weight": p + "mlp.router", "correction": p + "mlp.correction",
                 "gate_up_weight": Concat(tuple(e + w for e in experts for w in ("gate", "up")), dim=0),
                 "down_weight": Concat(tuple(e + "down" for e in experts), dim=0)}))
        if lc.mlp is not None:
            named["norm_feed_forward"] = ("norm", norm(p + "norm2"))
        if cfg.token_side_dim is not None:
            d = cfg.token_side_dim
            named["token_input"] = ("feed_forward", PartSpec(
                "token_gated_input",
                dict(hidden_size=width, dim=d, vocab_size=cfg.vocab, table_width=n_layers * d, column=i * d),
                {"table": "side.embed", "gate_weight": p + "side.gate", "proj_weight": p + "side.proj"}))
            named["norm_token_input"] = ("norm", norm(p + "side.norm"))
        block = PartSpec("normed_sublayers", dict(residual_mult=cfg.residual_mult, feed_forward=lc.mlp is not None,
                                                  token_input=cfg.token_side_dim is not None))
        layers.append(LayerSpec.of(block, **named))
    return ModelSpec(
        hidden_size=width,
        vocab_size=cfg.vocab,
        max_positions=cfg.max_positions,
        embedding=PartSpec("token_table", dict(vocab_size=cfg.vocab, hidden_size=width), {"weight": "embed"}),
        position=PartSpec("none"),
        layers=tuple(layers),
        run_order=tuple(RunEntry(i) for i in range(n_layers)),
        final_norm=norm("final.norm"),
        head=PartSpec("linear", dict(vocab_size=cfg.vocab, hidden_size=width), {"weight": "head"}),
        eos_token_id=cfg.eos_token_id,
    )


register_architecture("Lebedra", LebedraConfig, build_lebedra_spec, model_types=("lebedra",), replace=True)
