"""The Mogutar configuration, its description as parts and the cache's bookkeeping for it (no GPU)."""
import copy

import pytest
import torch

import mogutar_configs as C
import plain_mogutar as P
from rustyllm_b200 import ConfigError, resolve_architecture
from rustyllm_b200.cache.sequence_cache import KVNeed, SequenceCache
from rustyllm_b200.config.mogutar import MogutarConfig
from rustyllm_b200.models.decoder import DecoderModel
from rustyllm_b200.parts import Runtime
from rustyllm_b200.parts.rope import yarn_inverse_frequencies
from rustyllm_b200.weights.loader import check_checkpoint
from rustyllm_b200.weights.safetensors_io import Checkpoint


@pytest.mark.parametrize("name", list(C.CONFIGS) + list(range(12)))
def test_configuration_round_trip_and_tensor_names(tmp_path, name):
    cfg = C.CONFIGS[name] if isinstance(name, str) else C.random_config(name)
    arch = resolve_architecture(cfg)
    typed = arch.parse_config(cfg)
    assert isinstance(typed, MogutarConfig) and arch.parse_config(typed.to_dict()) == typed
    spec = arch.build_spec(typed)
    model = DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32))
    d = C.write_model(str(name), str(tmp_path / "m"), seed=1, cfg=cfg)
    check_checkpoint(model.param_specs(), Checkpoint(d).entries, spec.ignored_tensors, d)     # every tensor named, none left over
    # a parallel layer's entry: keys and values of the left mixer, state of both; a lightning layer: state alone
    for layer, (kv, state) in zip(cfg["layers"], model.entry_needs):
        if layer["type"] == "parallel":
            a, s = layer["mixer"]["left"], layer["mixer"]["right"]
            mask = a.get("mask") or {}
            assert kv == KVNeed(a["kv_heads"], a["dim"], mask.get("size"), a["vdim"], mask.get("keep_first", 0) if mask else 0)
            conv_left = 4 * (a.get("conv", 0) - 1) * ((a["heads"] + a["kv_heads"]) * a["dim"] + a["kv_heads"] * a["vdim"]) if a.get("conv", 0) > 1 else 0
            scan = 4 * s["heads"] * s["state"] * s["vdim"]
            assert state.nbytes >= conv_left + scan
        else:
            m = layer["mixer"]
            assert kv is None and state.nbytes == 4 * m["heads"] * m["dim"] * m["vdim"]


def test_configuration_errors_name_the_key():
    base = C.CONFIGS["T"]
    def broken(change):
        cfg = copy.deepcopy(base)
        change(cfg)
        return cfg
    cases = [
        (lambda c: c["layers"][0].__setitem__("type", "recurrent"), "mixer type"),
        (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3), "kv_heads"),
        (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("groups", 2), "groups"),
        (lambda c: c["layers"][0]["mlp"]["router"]["groups"].__setitem__("keep", 4), "groups"),
        (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 5), "top"),
        (lambda c: c["layers"][1]["mixer"].__setitem__("decay", [0.5]), "decay"),
        (lambda c: c["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 7), "dims"),
        (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "dense"), "kind"),
        (lambda c: c.pop("norm"), "norm"),
    ]
    for change, word in cases:
        with pytest.raises(ConfigError, match=word):
            MogutarConfig.from_dict(broken(change))


def test_stretched_frequencies_follow_the_plain_statement():
    for dims, base, sc in ((8, 10000.0, (2.0, 64, 8.0, 1.0)), (64, 1.0e6, (8.0, 4096, 32.0, 1.0)), (32, 300000.0, (4.0, 2048, 24.0, 1.0)),
                           (4, 100.0, (16.0, 100, 4.0, 0.5))):
        want, mult = P.yarn_frequencies(dims, base, dict(zip(("factor", "original", "fast", "slow"), sc)))
        got = yarn_inverse_frequencies(base, dims, *sc)
        torch.testing.assert_close(got.double(), torch.tensor(want, dtype=torch.float64), rtol=1e-6, atol=0)
        assert mult > 1.0


def test_window_pages_are_given_back_but_kept_first_tokens_stay():
    need = KVNeed(1, 8, window=70, keep_first=5)
    cache = SequenceCache([need, KVNeed(1, 8, window=70)], [None, None], 64 * 12, torch.float32, "cpu", max_slots=2)
    s = cache.alloc_slot()
    cache.prepare([s], [300])
    cache.commit([s], [300])
    kept, plain = cache.groups
    # the next query sits at 300 and reads from 231: pages 0..2 lie wholly in front of the window
    assert [p >= 0 for p in plain.slot_pages[s]] == [False, False, False, True, True]
    assert [p >= 0 for p in kept.slot_pages[s]] == [True, False, False, True, True]      # page 0 holds the kept tokens
    for _ in range(200):
        cache.prepare([s], [1])
        cache.commit([s], [1])
        cache.check()
    assert kept.slot_pages[s][0] >= 0 and sum(p >= 0 for p in kept.slot_pages[s]) == 3
    cache.free_slot(s)
    cache.check()
    assert kept.pages.held_count == 0 and plain.pages.held_count == 0
    assert KVNeed(1, 8, None, None, 9) == KVNeed(1, 8)          # without a window nothing is dropped anyway
