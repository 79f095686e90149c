"""Do the CPU cases of the Lokolorn suite notice faults?  One-line mutants of the scaled pre-norm arrangement, the pair of
mixers, the attention behind convolutions, both recurrences, the latent attention's new options, the routed feed-forward,
the loop entry and the configuration, applied in memory as in tests/test_mutants.py; a few of the suite's cases must fail
for each.  No GPU."""

import tempfile
from pathlib import Path

import pytest

from dli_b200.config import lokolorn as config_mod
from dli_b200.parts import base as base_mod
from dli_b200.parts import block as block_mod
from dli_b200.parts import entry as entry_mod
from dli_b200.parts.attention import ConvAttention, LatentAttention
from dli_b200.parts.mlp import RoutedGLU
from dli_b200.parts.pair import WeightedPairMixer
from dli_b200.parts.ssm import ChannelDeltaRule, ShiftDecayRecurrence
from tests import cpu_ops, lokolorn_suite as suite
from tests.test_mutants import mutate

DETECTORS = (suite.case_every_configuration_whole_prompt_and_layers, suite.case_prefill_then_token_by_token,
             suite.case_one_key_at_the_window_s_edge, suite.case_a_sink_takes_the_mass, suite.case_routing_follows_the_correction_and_the_groups)


def detect():
    for case in DETECTORS:
        with tempfile.TemporaryDirectory() as tmp, cpu_ops.patched():
            case(Path(tmp), "cpu", "float32")


MUTANTS = {
    "the mixer's scale is used for the feed-forward too": (block_mod.ScaledPreNormBlock, "forward", "self.scales[1])", "self.scales[0])"),
    "the feed-forward reads the mixer's norm": (block_mod.ScaledPreNormBlock, "forward", "y = normed_input(self.ffn_norm, stream.h, pending, self.ffn)",
                                                "y = normed_input(self.mixer_norm, stream.h, pending, self.ffn)"),
    "a scaled delta loses its second term": (base_mod.PendingScaled, "__init__", "self.a, self.fa, self.b, self.fb = out.a, out.fa, out.b, out.fb",
                                             "self.a, self.fa, self.b, self.fb = out.a, out.fa, None, 0.0"),
    "the two mixers swap their constants": (WeightedPairMixer, "forward", "WeightedPair(a, self.fa, b, self.fb)", "WeightedPair(a, self.fb, b, self.fa)"),
    "the second mixer gets the first one's state": (WeightedPairMixer, "forward", "states=cache.states[n:]", "states=cache.states[:n]"),
    "the attention's convolution has an activation": (ConvAttention, "forward", "activation=False)", "activation=True)"),
    "the attention's carried rows are not moved on": (ConvAttention, "forward", "if self.taps > 1:", "if False:"),
    "q and k are not divided by their root mean square": (ConvAttention, "forward", "self.rotary_dim, self.unit_eps, cache.page_size)", "self.rotary_dim, None, cache.page_size)"),
    "the output bias is left out": (ConvAttention, "forward", "return project_bias(out, self.wo, self.bo)", "return project_bias(out, self.wo, None)"),
    "the previous token's row is not kept": (ShiftDecayRecurrence, "forward", "ops.conv_state_update(shift, x, 0, batch.q_start, batch.state_slot)", "pass"),
    "the blends of r and k change places": (ShiftDecayRecurrence, "load", 'torch.stack([t["mu_" + s] for s in "rkvgw"], 0)', 'torch.stack([t["mu_" + s] for s in "krvgw"], 0)'),
    "the decay's tanh is left out": (ShiftDecayRecurrence, "forward", 'low = ops.activation(project(blends[4], w["w1"]), "tanh")', 'low = project(blends[4], w["w1"])'),
    "the recurrence takes the delta rule's update": (ShiftDecayRecurrence, "forward", '"bonus", w["u"]', '"delta", None'),
    "the delta rule's gate is SiLU": (ChannelDeltaRule, "forward", 'gate_after=True, gate="sigmoid")', "gate_after=True)"),
    "the decay reads the gate's inner product": (ChannelDeltaRule, "forward", "a = project(u[:, self.a_cols[0] : self.a_cols[1]],", "a = project(u[:, self.g_cols[0] : self.g_cols[1]],"),
    "the sinks are left out": (LatentAttention, "forward", "sink=self.sinks)", "sink=None)"),
    "cosines and sines keep their size": (LatentAttention, "forward", "amp=self.amp)", "amp=1.0)"),
    "neighbouring pairs are read as distant ones": (LatentAttention, "load", 'if self.pairing == "neighbours" and self.rotary_dim:', "if False:"),
    "the correction enters the weights": (cpu_ops, "moe_route", "w = s.gather(1, picked)", "w = choice.gather(1, picked)"),
    "a group is marked by its best expert alone": (cpu_ops, "moe_route", "topk(min(2, per), -1)", "topk(1, -1)"),
    "the router's scale is left out": (RoutedGLU, "forward", "self.group_keep, self.route_scale)", "self.group_keep, 1.0)"),
    "the loop entry forgets the embedding": (entry_mod.ConcatProject, "apply", "ops.concat_stream_rows(both, h, self.table, batch.token_ids)",
                                             "ops.concat_stream_rows(both, h, self.table, batch.token_ids * 0)"),
    "the window is read one token too wide": (config_mod, "_parse_latent", 'window = _positive(m["mask"]["size"], where + ".mask.size")',
                                              'window = _positive(m["mask"]["size"], where + ".mask.size") + 1'),
    "the kept groups are one more": (config_mod, "_parse_mlp", 'count, keep = _positive(r["groups"]["count"], where + ".router.groups.count"), _positive(r["groups"]["keep"], where + ".router.groups.keep")',
                                     'count, keep = _positive(r["groups"]["count"], where + ".router.groups.count"), min(_positive(r["groups"]["keep"], where + ".router.groups.keep") + 1, _positive(r["groups"]["count"], where))'),
}


@pytest.mark.timeout(300)
@pytest.mark.parametrize("name", list(MUTANTS), ids=lambda n: n.replace(" ", "_"))
def test_lokolorn_mutant_is_noticed(name, monkeypatch):
    owner, method, old, new = MUTANTS[name]
    mutate(monkeypatch, owner, method, old, new)
    if owner is cpu_ops:  # the stand-in table holds the function itself
        monkeypatch.setitem(cpu_ops.OPS, method, getattr(cpu_ops, method))
    with pytest.raises(Exception):  # a wrong number (AssertionError), or a folder that no longer loads
        detect()


def test_without_a_mutant_the_cases_pass():
    detect()
