"""The Pokadra model through the engine's host side on the CPU (float32, torch stand-ins for the kernels) against the
plain implementation; configuration parsing, run order and what the cache is asked to keep.  The GPU tests run the same
cases on the real kernels."""

import json
import warnings

import pytest

from dli_b200.cache import CacheManager, GroupSpec
from dli_b200.config.llama import UnsupportedModelError
from dli_b200.config.pokadra import PokadraConfig, pokadra_model_spec, pokadra_run_order
from tests import cpu_ops, pokadra_suite as suite


@pytest.mark.parametrize("case", suite.CASES, ids=lambda f: f.__name__[5:])
def test_case(case, tmp_path):
    with cpu_ops.patched():
        case(tmp_path, "cpu", "float32")


def test_run_order_and_what_the_cache_keeps():
    cfg = PokadraConfig.from_dict(suite.CONFIGS["readers"])
    order = pokadra_run_order(cfg)
    assert [(s.layer, s.cache_of) for s in order] == [(0, None), (1, 0), (2, None), (3, 0)]
    spec = pokadra_model_spec(cfg)
    owner = spec.layers[0].parts["mixer"].params
    # a reader without a window makes the owner's cache keep everything, whatever the owner's own mask is
    assert owner["window"] == 17 and owner["retain_window"] is None
    cfg = PokadraConfig.from_dict(suite.CONFIGS["mixed"])
    params = [layer.parts["mixer"].params for layer in pokadra_model_spec(cfg).layers]
    assert (params[0]["retain_window"], params[0]["retain_first"]) == (21, 5) and (params[0]["window"], params[0]["keep_first"]) == (13, 3)
    assert (params[4]["retain_window"], params[4]["own_kv"]) == (21, False) and params[2]["retain_window"] == 9


def test_pages_of_the_kept_first_tokens_are_never_given_back():
    m = CacheManager([GroupSpec(40, window=10, keep_first=9)], page_size=4, max_requests=2, enable_prefix_caching=False, watermark=0.0)
    m.allocate("a", list(range(50)))
    m.mark_computed("a", 50)
    table = m.block_table("a")
    assert all(p >= 0 for p in table[:3]) and all(p < 0 for p in table[3:10]) and all(p >= 0 for p in table[10:])
    m.check_invariants()
    m.free("a")
    m.check_invariants()


def test_configuration_is_checked():
    good = suite.CONFIGS["mixed"]
    parsed = PokadraConfig.from_dict(good)
    assert parsed.norm_groups == 3 and parsed.pair_table.buckets == 101 and parsed.layers[4].mixer.kv_from == 0 and parsed.token_side_dim == 6
    for path, value in ((("layers", 0, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "rot", "dims"), 7), (("layers", 0, "mixer", "rot", "dims"), 18),
                        (("layers", 0, "type"), "other"), (("layers", 0, "mlp", "kind"), "routed"), (("layers", 0, "mlp", "limit"), 0.0),
                        (("layers", 0, "mixer", "mask", "size"), 0), (("layers", 4, "mixer", "kv_from"), 1), (("layers", 4, "mixer", "kv_from"), 4),
                        (("layers", 4, "mixer", "dim"), 8), (("norm", "groups"), 5), (("layers", 1, "mixer", "width"), 0)):
        bad = json.loads(json.dumps(good))
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(UnsupportedModelError):
            PokadraConfig.from_dict(bad)
    bad = json.loads(json.dumps(good))
    del bad["layers"][0]["mixer"]["diff"]
    with pytest.raises(KeyError):
        PokadraConfig.from_dict(bad)
    extra = json.loads(json.dumps(good))
    extra["layers"][1]["mixer"]["surprise"] = 1
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        assert PokadraConfig.from_dict(extra) == parsed  # a key the parser does not know is reported, not obeyed
    assert any("surprise" in str(w.message) for w in seen)
    plainer = json.loads(json.dumps(good))
    del plainer["embedding"], plainer["token_side"], plainer["residual_mult"], plainer["norm"]["groups"]
    parsed = PokadraConfig.from_dict(plainer)
    assert parsed.pair_table is None and parsed.token_side_dim is None and parsed.residual_mult == 1.0 and parsed.norm_groups == 1 and parsed.embedding_scale == 1.0
