"""The Labolix decoder as a ``ModelSpec``: a token embedding; pre-norm layers (``prenorm_residual``)
whose norms are Dynamic Tanh (``dynamic_tanh``), each with one of three mixers -- grouped-query
attention with a sink whose score is 0 (``sink_attention``), latent attention with a sliding window
and a learned sink (``latent_attention``), or retention (``retention``) -- and a dense clamped gated
feed-forward (``clamped_glu``) or none; a final norm; a head tied to the embedding whose logits are
soft-capped.  Every mixer turns its queries and keys with a rotary encoding of its own (``rotary``).
A layer may run with another layer's tensors: the schedule then names that layer again, and the stop
keeps a cache or state of its own.  Tensor names: ``embed``, ``l<i>.norm1|norm2`` (with ``.b`` and
``.alpha``), ``l<i>.mix.*``, ``l<i>.mlp.gate|up|down``, ``final.norm``.
"""

from __future__ import annotations

from ..config.labolix_config import LabolixConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Labolix"
GLU_ALPHA = 1.702           # g * sigmoid(1.702 g)


def _rotary(rot, layout: str):
    if rot is None or rot.dims == 0:
        return PartSpec("rotary", dict(dims=0, base=1.0, layout=layout))
    return PartSpec("rotary", dict(dims=rot.dims, base=rot.base, layout=layout, scaling=rot.scaling_dict()))


def build_spec(cfg: LabolixConfig) -> ModelSpec:
    w = cfg.hidden_size
    norm = lambda name, optional=False: PartSpec("dynamic_tanh", dict(dim=w, name=name, optional=optional))
    layers, index = [], {}                      # index: the config's layer number -> place among the layers that have tensors
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        m = layer.mixer
        if layer.type == "attention":
            mixer = PartSpec("sink_attention", dict(hidden_size=w, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim,
                                                    value_dim=m.vdim, scale=m.scale, window=m.window, sink="zero"), "mix.")
            position = _rotary(m.rot, "interleaved")
        elif layer.type == "latent_attention":
            mixer = PartSpec("latent_attention", dict(hidden_size=w, num_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim,
                                                      value_dim=m.vdim, kv_rank=m.kv_rank, scale=m.scale, norm_eps=cfg.norm_eps,
                                                      window=m.window, sink="learned"), "mix.")
            position = _rotary(m.rot, "interleaved")
        else:
            mixer = PartSpec("retention", dict(hidden_size=w, num_heads=m.heads, head_dim=m.dim, value_dim=m.vdim, decay=m.decay,
                                               norm_eps=cfg.norm_eps), "mix.")
            position = _rotary(m.rot, "halves")
        ffn = None
        if layer.mlp is not None:
            ffn = PartSpec("clamped_glu", dict(hidden_size=w, intermediate_size=layer.mlp.ff, limit=layer.mlp.limit, alpha=GLU_ALPHA), "mlp.")
        # a layer without a feed-forward has no use for a second norm; a file that holds one all the same is accepted
        norms = (norm("norm1"), norm("norm2", optional=ffn is None))
        index[i] = len(layers)
        layers.append(LayerSpec(block="prenorm_residual", mixer=mixer, feed_forward=ffn, norms=norms, prefix=f"l{i}.", position=position))
    schedule = tuple(ScheduleEntry(index[i if layer.weights_of is None else layer.weights_of]) for i, layer in enumerate(cfg.layers))
    return ModelSpec(
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab_size, hidden_size=w, name="embed")),
        layers=tuple(layers),
        schedule=schedule,
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", dict(vocab_size=cfg.vocab_size, hidden_size=w, tied=True, tied_to="embed", name="head",
                                          softcap=cfg.logit_softcap)),
        position=PartSpec("token_index", dict()),
    )


register_architecture(ARCHITECTURE, LabolixConfig.from_dict, build_spec, replace=True)
