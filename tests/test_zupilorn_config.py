"""The Zupilorn configuration on the CPU: keys, the parts it names, tensor names and shapes, refusals."""

import pytest
import torch

import plain_zupilorn as plain
import zupilorn_cases as Z


def test_the_specification_names_every_tensor_the_plain_implementation_reads():
    from llm_pipeline_b200.config import resolve_config
    from llm_pipeline_b200.models import build_model

    for name, cfg in Z.CONFIGS.items():
        config = resolve_config(cfg)
        model = build_model(config)
        expected = {n: tuple(s.shape) for n, s in model.expected_params().items() if not s.optional}
        W = Z.weights_for(cfg, 0)
        assert expected == {n: tuple(t.shape) for n, t in W.items()}, name
        plain.forward(cfg, {k: v.double() for k, v in W.items()}, [1, 2, 3])       # and the oracle needs no other
        assert config.to_json()["layers"] == cfg["layers"]
        assert resolve_config(config.to_json()).model_spec() == config.model_spec()


def test_cache_needs_follow_the_layers():
    from llm_pipeline_b200.cache import StateSpec, TokenPagesSpec
    from llm_pipeline_b200.config import resolve_config
    from llm_pipeline_b200.models import build_model

    cfg = Z.CONFIGS["attention_first"]
    specs = build_model(resolve_config(cfg)).cache_specs()
    assert specs[0] == (TokenPagesSpec((36 + 8,), None), None)
    assert specs[1] == (None, StateSpec((2, 72), torch.float32))
    assert specs[3] == (TokenPagesSpec((24 + 4,), None), None)


@pytest.mark.parametrize("damage, message", [
    (lambda c: c["layers"][0].update(type="lstm"), "unknown type"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "lacks"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "router.top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "unknown mlp kind"),
    (lambda c: c.pop("norm"), "required keys"),
])
def test_refusals(damage, message):
    import copy
    from llm_pipeline_b200.config import resolve_config

    cfg = copy.deepcopy(Z.CONFIGS["hybrid"])
    damage(cfg)
    with pytest.raises(ValueError, match=message):
        resolve_config(cfg)


def test_a_random_model_folder_can_be_written_and_read_back(tmp_path):
    from llm_pipeline_b200.config import load_config
    from llm_pipeline_b200.models import build_model
    from llm_pipeline_b200.weights import write_random_model
    from llm_pipeline_b200.weights.source import SafetensorsSource, check_names_and_shapes

    folder = write_random_model(Z.CONFIGS["experts_only"], 3, str(tmp_path))
    config = load_config(folder)
    assert config.architecture == "Zupilorn"
    source = SafetensorsSource(folder)
    check_names_and_shapes(build_model(config).expected_params(), source)
    dwa = source.get("l1.dwa").float()
    assert dwa.shape == (3,) and abs(float(dwa.sum()) - 1.0) < 0.3          # about an average, not noise around zero
    source.close()
