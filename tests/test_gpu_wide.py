"""The engine at the layer widths of the full-size model (hidden 4096, 32 query heads over 8 kv heads
of 128, intermediate 12288, a vocabulary of 151936; two layers instead of thirty-six, which makes
no product smaller) against the plain implementation, in 32-bit and in bfloat16, under the same
cuttings as the tiny configurations: a prompt whole, its last 32 tokens one by one, and a batch of
unequal prompts whose shorter requests end earlier.  A prompt of 600 rows puts three to four tiles
on every CTA of the tiled tensor-core products of a layer; the reference gates its own full-size
path on an oracle in the same way (qwen3/official_test.go:92-118; internal/qwen3lm/weights_test.go:94-161).

The weights come from the library's seeded fill on the device.  That the fill is the function the
plain implementation restates is checked first, on whole small tensors and on sampled rows of every
large one; the plain forward pass then takes the values it is given.  The vocabulary is compared on
a sample of its columns (the first and last 128 and 4096 random ones): the oracle's head over all
151936 columns would take longer than everything else together.
"""
import numpy as np
import pytest
import torch

from tests.plain import qwen3_plain as P
from tests.test_gpu_replay import first_bad_row

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
SEED = 3


def wide_config():
    from gophonic_b200.config import Qwen3Config
    return Qwen3Config(hidden_size=4096, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                       intermediate_size=12288, vocab_size=151936, max_position_embeddings=4096, rms_norm_eps=1e-6,
                       rope_theta=1000000.0, tie_word_embeddings=False)


def to_host(t: torch.Tensor) -> np.ndarray:
    """float32 copy of a bfloat16 or float32 device tensor (exact)."""
    return t.detach().to(torch.float32).cpu().numpy()


@pytest.fixture(scope="module")
def wide():
    """dtype -> (engine, plain config, plain weights over the compact vocabulary, id maps)."""
    from gophonic_b200.engine import Engine, Model
    from gophonic_b200.engine.model import make_runtime
    from gophonic_b200.weights import random_tensors_on_device
    cfg = wide_config()
    spec = cfg.model_spec()
    pcfg = cfg.to_dict()
    rng = np.random.default_rng(17)
    V = cfg.vocab_size
    columns = np.unique(np.concatenate([np.arange(128), np.arange(V - 128, V), rng.integers(0, V, size=4096)]))
    made = {}

    def get(dtype):
        if dtype in made:
            return made[dtype]
        rt = make_runtime(dtype, DEV)
        tensors = random_tensors_on_device(spec, SEED, dtype, rt.device)
        # the fill on the device is the function the plain implementation restates
        shapes = P.tensor_shapes(pcfg)
        assert sorted(shapes) == sorted(tensors)
        pick = np.random.default_rng(5)
        for name, shape in shapes.items():
            t = tensors[name]
            assert tuple(t.shape) == tuple(shape)
            std, mean = (0.02, 1.0) if name.endswith("norm.weight") else (0.02, 0.0)
            if len(shape) == 1:
                assert np.array_equal(to_host(t), P.seeded_values(SEED, name, shape[0], std, mean)), name
                continue
            for r in np.unique(np.concatenate([[0, shape[0] - 1], pick.integers(0, shape[0], size=6)])):
                # element index = row * width + column: a row is a slice of the tensor's sequence
                want = P.seeded_values(SEED, name, shape[1], std, mean, first=int(r) * shape[1])
                assert np.array_equal(to_host(t[int(r)]), want), (name, int(r))
        # plain weights: the layers whole, the embedding and the head on the rows a test can touch
        w = {}
        for name, t in tensors.items():
            if name in ("model.embed_tokens.weight", "lm_head.weight"):
                continue
            w[name] = to_host(t)
        table = tensors["model.embed_tokens.weight"]
        head = tensors["lm_head.weight"]
        w["lm_head.weight"] = to_host(head[torch.from_numpy(columns).to(DEV)])
        model = Model(spec, tensors, rt, cfg)
        eng = Engine(model, max_tokens=4096)
        made[dtype] = (eng, pcfg, w, table, columns)
        return made[dtype]
    return get


_references = {}


def reference(wide_entry, tokens):
    """Plain logits [len(tokens), sampled columns] for one whole sequence (the weights hold the
    same values in both modes, so one evaluation serves both)."""
    key = tuple(tokens)
    if key not in _references:
        _, pcfg, w, table, _ = wide_entry
        ids, inverse = np.unique(np.asarray(tokens), return_inverse=True)
        ww = dict(w)
        ww["model.embed_tokens.weight"] = to_host(table[torch.from_numpy(ids).to(table.device)])
        _references[key] = P.forward_logits(inverse.tolist(), pcfg, ww)
    return _references[key]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_prompt_whole_and_its_last_32_tokens_one_by_one(wide, dtype):
    entry = wide(dtype)
    eng, pcfg, _, _, columns = entry
    rng = np.random.default_rng(23)
    toks = rng.integers(0, pcfg["vocab_size"], size=600).tolist()
    ref = reference(entry, toks)
    # whole: a sample of places, the first and the last among them
    places = sorted({0, 1, 63, 64, 127, 128, 255, 256, 511, 512, 598, 599} | set(rng.integers(0, 600, size=20).tolist()))
    slot = eng.new_sequence()
    got = eng.step([(slot, toks)], [places]).cpu().numpy()[:, columns]
    eng.end_sequence(slot)
    bad = first_bad_row(got, ref[places], dtype)
    assert bad is None, f"whole prompt: first wrong place {places[bad[0]]} ({bad[1]})"
    # the last 32 tokens one by one after the first 568 in one step
    slot = eng.new_sequence()
    out = [eng.step([(slot, toks[:568])], [[567]]).cpu().numpy()[:, columns]]
    for t in toks[568:]:
        out.append(eng.step([(slot, [t])]).cpu().numpy()[:, columns])
    eng.end_sequence(slot)
    bad = first_bad_row(np.concatenate(out, 0), ref[567:], dtype)
    assert bad is None, f"one by one: first wrong place {567 + bad[0]} ({bad[1]})"
    from gophonic_b200 import ops
    assert ops.tc5_status() == 0
    eng.cache.check()
    assert eng.cache.pages.held() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_batch_of_unequal_prompts_whose_shorter_requests_end_earlier(wide, dtype):
    entry = wide(dtype)
    eng, pcfg, _, _, columns = entry
    rng = np.random.default_rng(29)
    # the second batch uses the slots and pages again; the third decodes ten sequences together, where
    # the products of 9 to 64 rows carry the norms at these widths (32 tiles of 128 columns, 8 K slices)
    for plan in ([(150, 4), (40, 2), (70, 6)], [(9, 3), (300, 1)], [(2 + (7 * i) % 23, 2) for i in range(10)]):
        toks = [rng.integers(0, pcfg["vocab_size"], size=p + d).tolist() for p, d in plan]
        refs = [reference(entry, t) for t in toks]
        slots = [eng.new_sequence() for _ in plan]
        got = [[] for _ in plan]
        first = eng.step([(slots[i], toks[i][:p]) for i, (p, _) in enumerate(plan)], [[0, p - 1] for p, _ in plan]).cpu().numpy()[:, columns]
        for i in range(len(plan)):
            got[i].append(first[2 * i:2 * i + 2])
        for step in range(max(d for _, d in plan)):
            live = [i for i in range(len(plan)) if step < plan[i][1]]
            out = eng.step([(slots[i], [toks[i][plan[i][0] + step]]) for i in live]).cpu().numpy()[:, columns]
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
                if step + 1 >= plan[i][1]:
                    eng.end_sequence(slots[i])
        for i, (p, d) in enumerate(plan):
            places = [0, p - 1] + list(range(p, p + d))
            bad = first_bad_row(np.concatenate(got[i], 0), refs[i][places], dtype)
            assert bad is None, f"request {i} (prompt {p}, decoded {d}): first wrong place {places[bad[0]]} ({bad[1]})"
        eng.cache.check()
        assert eng.cache.pages.held() == 0 and eng.cache.slots.held() == 0


@pytest.mark.parametrize("mode", ["float32", "bfloat16"])
def test_the_device_fill_and_the_folder_writer_make_the_same_tensors(tmp_path, mode):
    """The same configuration and seed through ``write_random_model`` + the loader and through the
    fill kernel: equal dtypes and equal bits, tensor by tensor, tied and untied."""
    from tests.conftest import tiny_configs
    from gophonic_b200 import ops  # noqa: F401  (the library must be loaded for the device path)
    from gophonic_b200.weights import InitScales, declare_model, load_tensors, random_tensors_on_device, write_random_model
    scales = InitScales(matrix=0.1, embedding=1.0, head=0.3, norm=0.05)
    for name in ("A", "B"):
        cfg = tiny_configs()[name]
        spec = cfg.model_spec()
        d = str(tmp_path / name)
        write_random_model(cfg, seed=41, out_dir=d, weight_dtype="bfloat16", scales=scales)
        loaded = load_tensors(d, declare_model(spec), mode, DEV)
        made = random_tensors_on_device(spec, 41, mode, torch.device(DEV), scales, tied=cfg.tie_word_embeddings)
        assert sorted(loaded) == sorted(made)
        for k in loaded:
            assert loaded[k].dtype == made[k].dtype and torch.equal(loaded[k], made[k]), k
