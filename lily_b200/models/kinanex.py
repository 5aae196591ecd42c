"""The Kinanex decoder as a ``ModelSpec``.

The stream starts as the embedding rows under the model's RMS norm.  Every layer is a pre-norm block with a gain per
column behind each sublayer (a layer scale): ``x += s1 * mixer(norm1(x))`` and, where it has a feed-forward,
``x += s2 * ff(norm2(x))``.  The mixer is a gated delta-rule recurrence (``delta``), a selective scan with a state
vector per channel (``mamba1``), or a grouped-query softmax attention (``attention``) with biases, q/k norm, rotation
in halves with Llama-3 frequency scaling, values at unit root mean square that all layers but the first blend with the
first one's, one more unit in the softmax's denominator, and the heads' weights mixed by a matrix.  The feed-forward is
``down(g sigmoid(1.702 g) (u + 1))`` with clamped g and u.  The head is the embedding table; the logits are scaled.
Tensor names are the checkpoint's own (``l<i>.norm1``, ``l<i>.mix.q``, ``l<i>.ls1``, ``l<i>.mlp.gate``, ...).
"""

from __future__ import annotations

from lily_b200.config.kinanex_config import KinanexConfig
from lily_b200.config.registry import register_architecture
from lily_b200.parts.attention import AttentionSpec
from lily_b200.parts.base import ModelSpec, ScheduleEntry
from lily_b200.parts.block import SandwichBlockSpec
from lily_b200.parts.delta_rule import DeltaRuleSpec
from lily_b200.parts.mlp import SwiGLUSpec
from lily_b200.parts.norm import RMSNormSpec
from lily_b200.parts.rope import RopeSpec
from lily_b200.parts.selective_scan import SelectiveScanSpec

_ATTENTION_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("q_bias", "q.b"), ("k_bias", "k.b"), ("v_bias", "v.b"),
                    ("q_norm", "q.norm"), ("k_norm", "k.norm"), ("talk", "talk"), ("v_blend", "vmix"))
_FF_NAMES = (("gate", "gate"), ("up", "up"), ("down", "down"))
SWISH_ALPHA = 1.702            # the feed-forward's gate is g sigmoid(1.702 g)
UNIT_EPS = 1e-6                # inside the root that makes the delta rule's q and k unit vectors


def build_spec(cfg: KinanexConfig) -> ModelSpec:
    norm = RMSNormSpec(cfg.width, cfg.eps, suffix="")
    blocks, ignored = [], []
    shared_seen = False
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "delta":
            mixer = DeltaRuleSpec(cfg.width, m.heads, m.kv_heads, m.dim, m.vdim, m.conv, cfg.eps, unit_eps=UNIT_EPS)
        elif layer.type == "mamba1":
            mixer = SelectiveScanSpec(cfg.width, m.inner, m.state, m.dt_rank, m.conv)
        else:
            rope = RopeSpec(m.dim, m.rotary_dims, m.rotary_base, m.rotary_scaling, exact_frequencies=True) if m.rotary_dims else None
            share = None
            if m.v_mix:
                share, shared_seen = ("blend" if shared_seen else "first"), True
            mixer = AttentionSpec(cfg.width, m.heads, m.kv_heads, m.dim, qk_norm=True, norm_eps=cfg.eps, bias=True, out_bias=False,
                                  scale=m.scale, position=rope, v_head_dim=m.vdim, names=_ATTENTION_NAMES, sink=True,
                                  talk=True, v_norm=True, v_share=share)
            if not m.v_mix:
                ignored.append(f"l{i}.mix.vmix")             # a layer that shares no values has no use for the weight
        ff = None
        if layer.mlp is not None:
            ff = SwiGLUSpec(cfg.width, layer.mlp.ff, activation="swish_clamped", limit=layer.mlp.limit, alpha=SWISH_ALPHA,
                            names=_FF_NAMES)
        else:
            ignored += [f"l{i}.norm2", f"l{i}.ls2"]          # a layer without feed-forward has no use for these
        blocks.append(SandwichBlockSpec(prefix=f"l{i}", mixer=mixer, feed_forward=ff, norm=norm, post_divides=False,
                                        norm_names=("norm1", "ls1", "norm2", "ls2")))
    return ModelSpec(architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=cfg.width, blocks=blocks,
                     schedule=[ScheduleEntry(i) for i in range(len(blocks))], final_norm=norm, embed_name="embed",
                     final_norm_prefix="final.norm", head_name=None, max_position=cfg.max_positions,
                     ignored_tensors=tuple(ignored), logit_scale=cfg.logit_scale, embed_norm=norm, embed_norm_prefix="embed.norm")


register_architecture("Kinanex", KinanexConfig.from_dict, build_spec)
