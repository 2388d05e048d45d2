"""The Razelorn configuration on the CPU: keys, the parts it names, tensor names and shapes, the schedule of layers that
use another layer's tensors, refusals, and the rotation's frequency rescaling against the plain implementation."""

import copy

import pytest
import torch

import plain_razelorn as plain
import razelorn_cases as R


def test_the_specification_names_every_tensor_the_plain_implementation_reads():
    from llm_pipeline_b200.config import resolve_config
    from llm_pipeline_b200.models import build_model

    for name, cfg in R.CONFIGS.items():
        config = resolve_config(cfg)
        model = build_model(config)
        expected = {n: tuple(s.shape) for n, s in model.expected_params().items() if not s.optional}
        W = R.weights_for(cfg, 0)
        assert expected == {n: tuple(t.shape) for n, t in W.items()}, name
        plain.forward(cfg, {k: v.double() for k, v in W.items()}, [1, 2, 3])       # and the oracle needs no other
        assert config.to_json()["layers"] == cfg["layers"]
        assert resolve_config(config.to_json()).model_spec() == config.model_spec()


def test_layers_that_use_another_layers_tensors_run_its_parts_with_a_cache_of_their_own():
    from llm_pipeline_b200.cache import HeadRowPagesSpec
    from llm_pipeline_b200.config import resolve_config
    from llm_pipeline_b200.models import build_model

    model = build_model(resolve_config(R.CONFIGS["mixed"]))
    assert [(e.layer, e.cache) for e in model.schedule] == [(0, 0), (1, 1), (0, 2), (2, 3), (1, 4)]
    assert len(model.blocks) == 3
    specs = model.cache_specs()
    assert specs[0] == specs[2] == (HeadRowPagesSpec(2, 2 * 32 + 48, 24), None)
    assert specs[1] == specs[4] == (HeadRowPagesSpec(4, 2 * 16 + 16, None), None)
    assert specs[3] == (HeadRowPagesSpec(1, 2 * 64 + 32, 50), None)
    assert model.blocks[2].feed_forward is None


@pytest.mark.parametrize("damage, message", [
    (lambda c: c["layers"][0].update(type="lstm"), "unknown type"),
    (lambda c: c["layers"][1]["mixer"].pop("vdim"), "lacks"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=10), "router.top"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "unknown mlp kind"),
    (lambda c: c["layers"][2].update(weights_of=2), "weights_of"),
    (lambda c: c["layers"][2].update(weights_of=4), "weights_of"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=34), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(heads=7), "cannot share"),
    (lambda c: c.pop("norm"), "required keys"),
])
def test_refusals(damage, message):
    from llm_pipeline_b200.config import resolve_config

    cfg = copy.deepcopy(R.CONFIGS["mixed"])
    damage(cfg)
    with pytest.raises(ValueError, match=message):
        resolve_config(cfg)


def test_a_layer_that_uses_another_layers_tensors_is_described_by_that_layer():
    from llm_pipeline_b200.config import resolve_config

    cfg = copy.deepcopy(R.CONFIGS["mixed"])
    cfg["layers"][2] = {"type": "attention", "weights_of": 0}
    assert resolve_config(cfg).model_spec() == resolve_config(R.CONFIGS["mixed"]).model_spec()


def test_rescaled_frequencies_follow_the_plain_rule():
    from llm_pipeline_b200.parts.position import RotaryPositions

    for dims, base, rule in ((16, 10000.0, R.SCALING), (48, 500.0, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 300}),
                             (8, 100.0, {"factor": 2.0, "low": 2.0, "high": 3.0, "original": 50})):
        want = plain.rotary_frequencies(dims, base, rule)
        part = RotaryPositions("", dims, base, frequency_scaling=rule)
        assert torch.allclose(part._inv_freq_cpu.double(), want, rtol=1e-6, atol=0)
        kept = plain.rotary_frequencies(dims, base, None)
        # the rule must have done something to some frequency and left another alone, or the case tests nothing
        assert (want != kept).any() and (want == kept).any()
    assert torch.allclose(RotaryPositions("", 16, 10000.0)._inv_freq_cpu.double(), plain.rotary_frequencies(16, 10000.0, None), rtol=1e-6)


def test_a_random_model_folder_can_be_written_and_read_back(tmp_path):
    from llm_pipeline_b200.config import load_config
    from llm_pipeline_b200.models import build_model
    from llm_pipeline_b200.weights import write_random_model
    from llm_pipeline_b200.weights.source import SafetensorsSource, check_names_and_shapes

    folder = write_random_model(R.CONFIGS["shared_weights"], 3, str(tmp_path))
    config = load_config(folder)
    assert config.architecture == "Razelorn"
    source = SafetensorsSource(folder)
    check_names_and_shapes(build_model(config).expected_params(), source)
    assert "l1.norm1" not in source.names() and "l3.norm1.b" in source.names()
    assert abs(float(source.get("l0.norm1").float().mean()) - 1.0) < 0.2
    source.close()
