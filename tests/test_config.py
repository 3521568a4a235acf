import pytest
import torch

from agentgarten_b200.infra.config import (ConfigError, ConfigNode, LazyCall, apply_overrides,
                                            from_yaml, instantiate, locate, resolve, to_yaml)


def test_lazycall_records_defaults_and_instantiates():
    node = LazyCall(torch.nn.Linear)(in_features=3, out_features=2)
    assert node["_target_"] == "torch.nn.Linear" and node.bias is True
    layer = instantiate(node)
    assert isinstance(layer, torch.nn.Linear) and layer.weight.shape == (2, 3)
    assert instantiate(node, bias=False).bias is None  # runtime kwargs win


def test_overrides_grammar():
    cfg = ConfigNode({"a": {"b": 1, "c": [1, 2]}, "t": LazyCall(torch.nn.Linear)(in_features=1, out_features=1)})
    apply_overrides(cfg, ["a.b=2", "+a.new={x:1,y:[a,b]}", "++a.c=[3]", "t.bias=false", "~a.b"])
    assert "b" not in cfg.a and cfg.a.new.y == ["a", "b"] and cfg.a.c == [3] and cfg.t.bias is False
    with pytest.raises(ConfigError):
        apply_overrides(cfg, ["a.missing=1"])
    with pytest.raises(ConfigError):
        apply_overrides(cfg, ["+a.c=1"])
    apply_overrides(cfg, ["t={_target_:torch.nn.Identity}"])
    assert isinstance(instantiate(cfg.t), torch.nn.Identity)
    apply_overrides(cfg, ["a.new=null"])
    assert cfg.a.new is None


def test_interpolation_env_and_missing(monkeypatch):
    monkeypatch.setenv("AGB_TEST_ROOT", "/data")
    cfg = ConfigNode({"paths": {"root": "${oc.env:AGB_TEST_ROOT,/tmp}", "other": "${oc.env:AGB_NOPE,fallback}"},
                      "out": "${paths.root}/run", "dup": "${paths}", "need": "???"})
    with pytest.raises(ConfigError):
        resolve(cfg)
    cfg.need = 1
    done = resolve(cfg)
    assert done.out == "/data/run" and done.paths.other == "fallback" and done.dup.root == "/data"
    again = from_yaml(to_yaml(done))
    assert again == done
    with pytest.raises(ConfigError):
        resolve(ConfigNode({"a": "${b}", "b": "${a}"}))


def test_locate_errors():
    assert locate("torch.nn.Linear") is torch.nn.Linear
    with pytest.raises(ImportError):
        locate("torch.nn.DoesNotExist")
    with pytest.raises(ImportError):
        locate("nodots")


def test_dataclass_nodes_roundtrip():
    from agentgarten_b200.networks.cosmos3 import Cosmos3Config

    cfg = ConfigNode({"c": LazyCall(Cosmos3Config)(hidden_size=64)})
    built = instantiate(resolve(cfg)).get("c") if isinstance(instantiate(resolve(cfg)), dict) else None
    assert isinstance(built, Cosmos3Config) and built.hidden_size == 64 and built.mrope_section == (24, 20, 20)
