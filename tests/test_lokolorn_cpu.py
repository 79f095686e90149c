"""The Lokolorn model through the engine's host side on the CPU (float32, torch stand-ins for the kernels) against the plain
implementation; configuration parsing and run order.  The GPU tests run the same cases on the real kernels."""

import json
import warnings

import pytest

from dli_b200.config.llama import UnsupportedModelError
from dli_b200.config.lokolorn import LokolornConfig, lokolorn_run_order
from dli_b200.config.registry import resolve_architecture
from tests import cpu_ops, lokolorn_suite as suite
from tests.plain import lokolorn_plain as plain


@pytest.mark.parametrize("case", suite.CASES, ids=lambda f: f.__name__[5:])
def test_case(case, tmp_path):
    with cpu_ops.patched():
        case(tmp_path, "cpu", "float32")


def test_run_order_follows_the_loop():
    for name, cfg in suite.CONFIGS.items():
        parsed = resolve_architecture(cfg).parse_config(cfg)
        order = lokolorn_run_order(parsed)
        start = (cfg.get("loop") or {}).get("start")
        assert [(s.layer, s.entry) for s in order] == [(i, t if i == start else None) for i, t in plain.layer_runs(cfg)], name
        assert all(s.cache_of is None for s in order)  # every pass keeps a cache and a state of its own


def test_configuration_is_checked():
    good = suite.CONFIGS["mixed_loop"]
    parsed = LokolornConfig.from_dict(good)
    assert isinstance(parsed, LokolornConfig) and parsed.layers[2].mixer.window == 13 and parsed.layers[0].mixer.left_scale == 0.9
    assert parsed.layers[0].mlp.group_count == 3 and parsed.layers[0].mlp.group_keep == 2 and parsed.layers[2].mixer.rot.scaling[0] == 4.0
    for path, value in ((("layers", 1, "mixer", "kv_heads"), 3), (("layers", 2, "mixer", "rot", "dims"), 7), (("layers", 2, "mixer", "rot", "dims"), 10),
                        (("layers", 0, "type"), "other"), (("loop", "stop"), 9), (("loop", "times"), 0), (("layers", 0, "mlp", "kind"), "dense"),
                        (("layers", 2, "mixer", "mask", "size"), 0), (("layers", 1, "mixer", "conv"), 0), (("layers", 0, "mixer", "left", "kv_heads"), 3),
                        (("layers", 0, "mlp", "router", "groups", "count"), 4), (("layers", 0, "mlp", "router", "top"), 5),
                        (("layers", 0, "mlp", "router", "groups", "keep"), 4), (("layers", 0, "mixer", "left", "rot", "dims"), 18)):
        bad = json.loads(json.dumps(good))
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(UnsupportedModelError):
            LokolornConfig.from_dict(bad)
    bad = json.loads(json.dumps(good))
    del bad["layers"][0]["mixer"]["right_scale"]
    with pytest.raises(KeyError):
        LokolornConfig.from_dict(bad)
    extra = json.loads(json.dumps(good))
    extra["layers"][1]["mixer"]["surprise"] = 1
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        assert LokolornConfig.from_dict(extra) == parsed  # a key the parser does not know is reported, not obeyed
    assert any("surprise" in str(w.message) for w in seen)
    plainer = json.loads(json.dumps(good))
    del plainer["loop"], plainer["layers"][0]["mlp"]["router"]["groups"], plainer["layers"][1]["mixer"]["decay_rank"]
    parsed = LokolornConfig.from_dict(plainer)
    assert parsed.loop is None and parsed.layers[0].mlp.group_count == 1 and parsed.layers[1].mixer.decay_rank is None


def test_sizes_left_to_the_checkpoint_are_read_from_it(tmp_path):
    """The inner sizes of the low-rank products are given by no key: a folder written with them loads through a configuration without."""
    import dli_b200

    cfg = suite.CONFIGS["mixed_loop"]
    suite.make_model(tmp_path / "m", cfg, seed=1)
    bare = json.loads(json.dumps(cfg))
    del bare["layers"][0]["mixer"]["right"]["decay_rank"], bare["layers"][1]["mixer"]["decay_rank"], bare["layers"][1]["mixer"]["gate_rank"]
    (tmp_path / "m" / "config.json").write_text(json.dumps(bare))
    with cpu_ops.patched():
        model = dli_b200.load_model(tmp_path / "m", "float32", "cpu")
    assert model.layers[1].mixer.a_cols[1] - model.layers[1].mixer.a_cols[0] == 5
