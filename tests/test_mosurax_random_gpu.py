"""Mosurax configurations drawn at random, every size free (tests/mosurax_configs.random_config), in both
dtypes against the plain implementation: whole, a prompt and then token by token, and as a batch of unequal
prompts decoded together."""
import os

import pytest
import torch

import mosurax_configs as C
import plain_mosurax as P
from gpu_helpers import random_tokens
from test_mosurax_gpu import close

pytestmark = pytest.mark.gpu
SEEDS = list(range(int(os.environ.get("MOSURAX_RANDOM_CONFIGS", "14"))))      # more for a long run


@pytest.mark.parametrize("seed", SEEDS)
def test_random_configuration(tmp_path, seed):
    from rustyllm_b200 import Runner
    cfg = C.random_config(seed)
    d = C.write_model(None, str(tmp_path / "m"), seed=1000 + seed, cfg=cfg)
    _, w = P.load_model_dir(d)
    V = cfg["vocab"]
    seqs = [random_tokens(V, n, 50 * seed + i) for i, n in enumerate((140, 9, 70))]
    refs = [P.forward(cfg, w, s) for s in seqs]
    for dtype in ("float32", "bfloat16"):
        r, _ = Runner.from_path(d, dtype=dtype, max_cache_tokens=64 * 8, max_batch=4)
        eng = r.engine
        # whole
        s = eng.alloc_slot()
        close(eng.step([s], [seqs[0]], "all"), refs[0], dtype, cfg, f"seed {seed} whole")
        eng.free_slot(s)
        # a prompt, then token by token (the captured step after the first)
        s = eng.alloc_slot()
        rows = [eng.step([s], [seqs[0][:100]], "all")] + [eng.step([s], [[t]], "last") for t in seqs[0][100:]]
        eng.free_slot(s)
        close(torch.cat(rows), refs[0], dtype, cfg, f"seed {seed} token by token")
        # a batch of unequal prompts, decoded together, the shorter ending earlier
        cut = [100, 4, 30]
        slots = [eng.alloc_slot() for _ in seqs]
        out = eng.step(slots, [q[:c] for q, c in zip(seqs, cut)], "all")
        got, o = [], 0
        for c in cut:
            got.append([out[o:o + c]])
            o += c
        at = list(cut)
        live = [0, 1, 2]
        while live:
            out = eng.step([slots[i] for i in live], [[seqs[i][at[i]]] for i in live], "last")
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
                at[i] += 1
            for i in [i for i in live if at[i] == len(seqs[i])]:
                eng.free_slot(slots[i])
            live = [i for i in live if at[i] < len(seqs[i])]
        for i in range(3):
            close(torch.cat(got[i]), refs[i], dtype, cfg, f"seed {seed} batch request {i}")
        r.cache.check()
        assert r.cache.free_pages == r.cache.num_pages
