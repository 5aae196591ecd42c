"""The Gotivik decoder as a ``ModelSpec``.

Every layer is a sandwich block: ``x += m * norm1b(mixer(norm1(x)))`` and, where it has a feed-forward,
``x += m * norm2b(ff(norm2(x)))``, with ``m`` one multiplier for the model.  The mixer is a grouped-query softmax attention
whose q, k and v pass a short causal convolution before q and k are rotated (halves, YaRN-scaled frequencies), over
a window that keeps a request's first positions in sight (``attention``); or a differential attention with a query
temperature by position, capped scores and a gate per head (``attention_2``).  The feed-forward is
``down(relu(up x)^2)``.  A layer that names another with ``weights_of`` is a second run of that layer's block in the
schedule, with a cache and state of its own.  The head is the embedding table.  Tensor names are the checkpoint's own
(``l<i>.norm1``, ``l<i>.mix.q``, ``l<i>.mix.q.conv``, ``l<i>.mlp.up``, ...).
"""

from __future__ import annotations

from lily_b200.config.gotivik_config import ConvAttentionConfig, GotivikConfig
from lily_b200.config.registry import register_architecture
from lily_b200.parts.attention import AttentionSpec
from lily_b200.parts.base import ModelSpec, ScheduleEntry
from lily_b200.parts.block import SandwichBlockSpec
from lily_b200.parts.diff_attention import DiffAttentionSpec
from lily_b200.parts.mlp import DenseMLPSpec
from lily_b200.parts.norm import RMSNormSpec
from lily_b200.parts.rope import RopeSpec

_ATTENTION_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("q_conv", "q.conv"), ("k_conv", "k.conv"), ("v_conv", "v.conv"))
_DIFF_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("g", "g"), ("lq1", "lq1"), ("lk1", "lk1"), ("lq2", "lq2"), ("lk2", "lk2"))
_FF_NAMES = (("up", "up"), ("down", "down"))


def build_spec(cfg: GotivikConfig) -> ModelSpec:
    norm = RMSNormSpec(cfg.width, cfg.eps, suffix="")
    blocks, block_of, ignored = [], {}, []
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        m = layer.mixer
        if isinstance(m, ConvAttentionConfig):
            rope = RopeSpec(m.dim, m.rotary_dims, m.rotary_base, m.rotary_scaling, exact_frequencies=True) if m.rotary_dims else None
            mixer = AttentionSpec(cfg.width, m.heads, m.kv_heads, m.dim, norm_eps=cfg.eps, window=m.window, scale=m.scale,
                                  position=rope, v_head_dim=m.vdim, names=_ATTENTION_NAMES,
                                  keep_first=m.keep_first if m.window else 0, conv_taps=m.conv)
        else:
            mixer = DiffAttentionSpec(cfg.width, m.heads, m.kv_heads, m.dim, m.vdim, m.scale, m.diff, cfg.eps,
                                      softcap=m.softcap, q_temp_coef=m.q_temp_coef, q_temp_every=m.q_temp_every,
                                      names=_DIFF_NAMES)
        ff = None if layer.ff is None else DenseMLPSpec(cfg.width, layer.ff, activation="relu2", names=_FF_NAMES)
        if ff is None:
            ignored += [f"l{i}.norm2", f"l{i}.norm2b"]      # a layer without feed-forward has no use for these gains
        block_of[i] = len(blocks)
        blocks.append(SandwichBlockSpec(prefix=f"l{i}", mixer=mixer, feed_forward=ff, norm=norm, mult=cfg.residual_mult))
    schedule = [ScheduleEntry(block_of[cfg.owner(i)]) for i in range(len(cfg.layers))]
    return ModelSpec(architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=cfg.width, blocks=blocks,
                     schedule=schedule, final_norm=norm, embed_name="embed", final_norm_prefix="final.norm", head_name=None,
                     max_position=cfg.max_positions, ignored_tensors=tuple(ignored))


register_architecture("Gotivik", GotivikConfig.from_dict, build_spec)
