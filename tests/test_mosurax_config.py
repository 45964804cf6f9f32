"""Mosurax on the CPU: its configuration, its description as parts, its tensors, and the plain
implementation's own mechanisms on values worked out by hand."""
import copy
import math

import pytest
import torch

import mosurax_configs as C
import plain_mosurax as P
from rustyllm_b200.config.files import ConfigError
from rustyllm_b200.config.mosurax import MosuraxConfig
from rustyllm_b200.config.registry import resolve_architecture
from rustyllm_b200.weights.loader import WeightsError, check_checkpoint
from rustyllm_b200.weights.random_init import _model_param_specs, write_random_model
from rustyllm_b200.weights.safetensors_io import Checkpoint


@pytest.mark.parametrize("name", list(C.CONFIGS))
def test_configuration_round_trip_and_schedule(name):
    d = C.CONFIGS[name]
    arch = resolve_architecture(d)
    cfg = arch.parse_config(d)
    assert isinstance(cfg, MosuraxConfig) and cfg.to_dict() == d
    spec = arch.build_spec(cfg)
    n, loop = len(d["layers"]), d.get("loop")
    want = list(range(n))
    if loop:
        want = list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"] + list(range(loop["stop"], n))
    assert list(spec.schedule) == want
    if loop:
        assert [(i.before_run, i.args["row"], i.args["again"]) for i in spec.injections] == \
            [(loop["start"] + t * (loop["stop"] - loop["start"]), t, t > 0) for t in range(loop["times"])]
    else:
        assert not spec.injections and not spec.inject_parts
    for l, ls in zip(d["layers"], spec.layers):
        m = ls.mixer.params
        assert (m["num_heads"], m["num_kv_heads"], m["head_dim"], m["value_dim"], m["scale"]) == \
            (l["mixer"]["heads"], l["mixer"]["kv_heads"], l["mixer"]["dim"], l["mixer"]["vdim"], l["mixer"]["scale"])
        assert m["window"] == (l["mixer"]["mask"]["size"] if "mask" in l["mixer"] else None) and m["sink"] is True
        assert ls.feed_forward.kind == {"dense": "gated_mlp", "moe": "moe_mlp"}.get((l["mlp"] or {}).get("kind"), "none")
    assert spec.head.params["softcap"] == d.get("logit_softcap")


def test_every_layer_run_gets_a_cache_of_its_own():
    from rustyllm_b200.models.decoder import DecoderModel
    from rustyllm_b200.parts import Runtime
    d = C.CONFIGS["P"]
    arch = resolve_architecture(d)
    model = DecoderModel(arch.build_spec(arch.parse_config(d)), Runtime(torch.device("cpu"), torch.float32))
    assert len(model.entry_needs) == len(model.spec.schedule) == 8
    assert [e for e, _ in model.run_entry] == list(range(8)) and all(w for _, w in model.run_entry)


def test_tensor_names_and_shapes(tmp_path):
    for name in C.CONFIGS:
        d = C.write_model(name, str(tmp_path / name))
        cfg = C.CONFIGS[name]
        arch = resolve_architecture(cfg)
        spec = arch.build_spec(arch.parse_config(cfg))
        ck = Checkpoint(d)
        check_checkpoint(_model_param_specs(cfg), ck.entries, spec.ignored_tensors, d)
        assert {n: tuple(e.shape) for n, e in ck.entries.items()} == C.tensor_shapes(cfg)
    # a missing tensor and a wrong shape are named
    bad = copy.deepcopy(C.CONFIGS["P"])
    bad["layers"][1]["mlp"]["router"]["experts"] = 6
    with pytest.raises(WeightsError) as e:
        check_checkpoint(_model_param_specs(bad), Checkpoint(str(tmp_path / "P")).entries, (), "x")
    assert "l1.mlp.e5.gate" in e.value.missing and any(n == "l1.mlp.router" for n, _, _ in e.value.wrong_shape)


def test_random_model_folder_of_the_library_fits_the_plain_reader(tmp_path):
    d = write_random_model(str(tmp_path / "m"), C.CONFIGS["S"], seed=3, dtype="bfloat16")
    cfg, w = P.load_model_dir(d)
    assert set(w) == set(C.tensor_shapes(cfg))
    assert P.forward(cfg, w, [1, 2, 3]).shape == (3, cfg["vocab"])


@pytest.mark.parametrize("change,needle", [
    (lambda d: d["layers"][0].update(type="recurrent"), "mixer type"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda d: d["layers"][0]["mlp"].update(kind="other"), "kind"),
    (lambda d: d["loop"].update(stop=9), "loop"),
    (lambda d: d.update(logit_softcap=-1.0), "logit_softcap"),
    (lambda d: d.pop("vocab"), "vocab"),
])
def test_configuration_errors_say_what_is_wrong(change, needle):
    d = copy.deepcopy(C.CONFIGS["P"])
    change(d)
    with pytest.raises(ConfigError) as e:
        MosuraxConfig.from_dict(d)
    assert needle in str(e.value)


def test_plain_mechanisms_on_values_worked_out_by_hand():
    assert P.sink_softmax([0.0]) == [0.5]
    p = P.sink_softmax([math.log(3.0), 0.0])
    assert abs(p[0] - 0.6) < 1e-12 and abs(p[1] - 0.2) < 1e-12
    # two tokens, window 1: each sees only itself; score 0 -> half of its own value
    q = torch.zeros(2, 1, 2, dtype=torch.float64)
    k = torch.ones(2, 1, 2, dtype=torch.float64)
    v = torch.tensor([[[2.0]], [[4.0]]], dtype=torch.float64)
    assert P.windowed_sink_attention(q, k, v, 1.0, 1).flatten().tolist() == [1.0, 2.0]
    # window 2: the second token sees both, three equal terms with the sink
    assert abs(float(P.windowed_sink_attention(q, k, v, 1.0, 2)[1, 0, 0]) - 2.0) < 1e-12
    chosen, weights = P.route(torch.tensor([0.0, 2.0, 2.0, 1.0], dtype=torch.float64), 2)
    assert chosen == [1, 2] and weights == [0.5, 0.5]
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(P.rms_norm(x, torch.ones(2, dtype=torch.float64), 0.0), x / math.sqrt(12.5))
    assert abs(float(P.soft_cap(torch.tensor([1e9], dtype=torch.float64), 5.0)) - 5.0) < 1e-9


def test_command_line_inspects_a_folder(tmp_path, capsys):
    from rustyllm_b200 import cli
    d = C.write_model("S", str(tmp_path / "S"))
    assert cli.main([d, "--inspect", "--list-tensors"]) == 0
    out = capsys.readouterr().out
    assert "architecture: Mosurax" in out and "compatibility: supported" in out and "l1.mlp.e6.down" in out and "width: 48" in out
