"""The Rirulix decoder as a ``ModelSpec``: a token embedding with learned positions and a norm;
layers whose sublayers are normalised before and after (``sandwich_residual``), each with a gated
linear recurrence (``rglru``) or attention with a distance bias, a window beside kept first tokens
and values mixed with the first such layer's (``biased_window_attention``), and a routed
feed-forward (``routed_glu``) or none; a final norm and an untied head.  All norms are RMS norms in
groups.  Tensor names: ``embed``, ``pos``, ``embed.norm``, ``l<i>.norm1|norm1b|norm2|norm2b``,
``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.rirulix_config import RirulixConfig
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Rirulix"
RGLRU_GAIN = 8.0            # log a = -8 r softplus(lam)
GLU_ALPHA = 1.702           # g * sigmoid(1.702 g)


def build_spec(cfg: RirulixConfig) -> ModelSpec:
    h = cfg.hidden_size
    norm = lambda name, optional=False: PartSpec("rmsnorm", dict(dim=h, eps=cfg.norm_eps, groups=cfg.norm_groups, name=name,
                                                                 optional=optional))
    layers = []
    value_source = None                 # (kv heads, value size) of the first layer that mixes values
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "attention":
            value_mix = None
            if m.v_mix:
                value_mix = "follower" if value_source else "source"
                if value_source and value_source != (m.kv_heads, m.vdim):
                    raise ValueError(f"layers[{i}] mixes its values ({m.kv_heads} heads of {m.vdim}) with those of the first "
                                     f"such layer, which has {value_source[0]} heads of {value_source[1]}")
                value_source = value_source or (m.kv_heads, m.vdim)
            mixer = PartSpec("biased_window_attention", dict(
                hidden_size=h, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim, scale=m.scale,
                window=m.window, keep_first=m.keep_first, distance_bias=True, value_mix=value_mix), "mix.")
        else:
            mixer = PartSpec("rglru", dict(hidden_size=h, width=m.width, blocks=m.blocks, conv=m.conv, gain=RGLRU_GAIN), "mix.")
        ffn = None
        names = ["norm1", "norm1b"]
        unused = ["norm2", "norm2b"]         # of a layer without a feed-forward: accepted in a file, never run
        if layer.mlp is not None:
            f = layer.mlp
            ffn = PartSpec("routed_glu", dict(hidden_size=h, experts=f.experts, top=f.top, expert_size=f.ff, limit=f.limit,
                                              alpha=GLU_ALPHA, shared_size=f.shared_ff, shared_limit=f.shared_limit), "mlp.")
            names, unused = names + unused, []
        layers.append(LayerSpec(block="sandwich_residual", mixer=mixer, feed_forward=ffn,
                                norms=tuple(norm(n) for n in names) + tuple(norm(n, True) for n in unused), prefix=f"l{i}."))
    return ModelSpec(
        embedding=PartSpec("learned_position_embedding", dict(vocab_size=cfg.vocab_size, hidden_size=h, max_positions=cfg.max_positions,
                                                              norm_eps=cfg.norm_eps, norm_groups=cfg.norm_groups,
                                                              names=("embed", "pos", "embed.norm"))),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", dict(vocab_size=cfg.vocab_size, hidden_size=h, tied=False, name="head")),
        position=PartSpec("token_index", dict(limit=cfg.max_positions)),
    )


register_architecture(ARCHITECTURE, RirulixConfig.from_dict, build_spec, replace=True)
