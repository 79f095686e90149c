"""Do the CPU cases of the Sugonex suite notice faults?  One-line mutants of the side-by-side arrangement, the
attention over a cached latent, the delta rule mixer, the norm pair, the head and the configuration, applied in
memory as in tests/test_mutants.py; a few of the suite's cases must fail for each.  No GPU."""

import tempfile
from pathlib import Path

import pytest

from dli_b200.config import sugonex as config_mod
from dli_b200.parts import block as block_mod
from dli_b200.parts import model as model_mod
from dli_b200.parts import norm as norm_mod
from dli_b200.parts.attention import LatentAttention
from dli_b200.parts.base import ResidualStream
from dli_b200.parts.ssm import GatedDeltaRule
from tests import cpu_ops, sugonex_suite as suite
from tests.test_mutants import mutate

DETECTORS = (suite.case_every_configuration_whole_prompt_and_layers, suite.case_prefill_then_token_by_token,
             suite.case_one_key_at_the_window_s_edge, suite.case_the_soft_cap_bends_large_logits)


def detect():
    for case in DETECTORS:
        with tempfile.TemporaryDirectory() as tmp, cpu_ops.patched():
            case(Path(tmp), "cpu", "float32")


MUTANTS = {
    "the feed-forward reads the mixer's norm": (block_mod.ParallelBlock, "forward", "ya, yf = ys", "ya, yf = ys[0], ys[0]"),
    "the feed-forward's output is not added": (block_mod.ParallelBlock, "forward", "PendingSum(a, self.ffn.forward(yf) if self.has_ffn else None)", "PendingSum(a, None)"),
    "the pair of outputs of the layer before is forgotten": (block_mod.ParallelBlock, "forward", "ys = pair(stream.h, stream.take_pending(), self.ffn_norm)", "ys = pair(stream.h, None, self.ffn_norm)"),
    "a pending pair loses its second half when settled": (ResidualStream, "settle", "self.h += delta.total()", "self.h += delta.a.float()"),
    "the norm's weight is not offset": (norm_mod.RMSNorm, "load", "tensors[self.name] + self.offset if self.offset else tensors[self.name]", "tensors[self.name]"),
    "the second norm of a pair uses the first one's weight": (norm_mod.RMSNorm, "add_norm_pair", "self.weight, other.weight, self.eps, None)", "self.weight, self.weight, self.eps, None)"),
    "the attention ignores the window": (LatentAttention, "forward", "self.nh, self.scale, self.window, splits=", "self.nh, self.scale, None, splits="),
    "the latent space queries use the value matrix": (LatentAttention, "forward", "[:, :, : self.d], self.w_uk,", "[:, :, : self.d], self.w_uv.transpose(1, 2)[:, : self.d, :] if self.dv >= self.d else self.w_uk,"),
    "the output gate is left out": (LatentAttention, "forward", "if self.gated else None)", "if False else None)"),
    "the rotated part does not rotate": (LatentAttention, "forward", "self.nh, self.d, self.dr, self.rank, self.rotary_dim, cache.page_size, amp=self.amp)", "self.nh, self.d, self.dr, self.rank, 0, cache.page_size, amp=self.amp)"),
    "beta and the decay change places": (GatedDeltaRule, "forward", "self.b_col, self.a_col, w[", "self.a_col, self.b_col, w["),
    "the convolution's carried inputs are not moved on": (GatedDeltaRule, "forward", "if self.taps > 1:", "if False:"),
    "the gate enters the norm": (GatedDeltaRule, "forward", "gate_after=True", "gate_after=False"),
    "query and key taps change places": (GatedDeltaRule, "load", 'torch.cat([t["q_conv"], t["k_conv"], t["v_conv"]], 0)', 'torch.cat([t["k_conv"], t["q_conv"], t["v_conv"]], 0)'),
    "the soft cap is not applied": (model_mod.LMHead, "forward", "ops.scale_softcap(logits, self.scale, self.softcap)", "ops.scale_softcap(logits, self.scale, 0.0)"),
    "the logit factor is not applied": (model_mod.LMHead, "forward", "ops.scale_softcap(logits, self.scale, self.softcap)", "ops.scale_softcap(logits, 1.0, self.softcap)"),
    "the window is read one token too wide": (config_mod, "_parse_latent", 'window = _positive(m["mask"]["size"], where + ".mask.size")', 'window = _positive(m["mask"]["size"], where + ".mask.size") + 1'),
    "the two kinds of attention swap their gates": (config_mod, "_parse_latent", "base, dims, window, gate)", "base, dims, window, not gate)"),
}


@pytest.mark.timeout(300)
@pytest.mark.parametrize("name", list(MUTANTS), ids=lambda n: n.replace(" ", "_"))
def test_sugonex_mutant_is_noticed(name, monkeypatch):
    owner, method, old, new = MUTANTS[name]
    mutate(monkeypatch, owner, method, old, new)
    with pytest.raises(Exception):  # a wrong number (AssertionError), or a folder that no longer loads
        detect()


def test_without_a_mutant_the_cases_pass():
    detect()
