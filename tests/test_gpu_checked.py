"""The build with bounds-checked indices (GOPHONIC_B200_CHECKED=1), in a process of its own: the
stand-in for a memory checker where none can be run.  Its kernels hold every index into the block
table, a cache plane, the embedding table or a token source against its bound before they use it;
an index out of bounds is recorded and the access skipped or redirected to element 0.

Two things are shown.  The engine's own steps (prompts, single tokens, unequal batches, a rewind, the
tcgen05 kernels of a head size of 128) trip no check and give the plain implementation's logits.
And indices that are wrong on purpose are caught, each with its value and bound, while the kernel
runs to its end: this part only runs after the process has made sure that it did load the checked
library, so a wrong index never reaches an unchecked kernel.
"""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r'''
import json, os, sys, tempfile
import numpy as np
import torch
sys.path.insert(0, os.getcwd())
from gophonic_b200 import ops
assert ops.is_checked_build(), "the checked library was not loaded"
from gophonic_b200.engine import Engine, Model
from gophonic_b200.weights import InitScales, write_random_model
from tests.conftest import tiny_configs
from tests.plain import qwen3_plain as P

report = {"checked": True, "clean": [], "caught": {}}
DEV = "cuda:0"

# ---- the engine's own steps trip nothing -----------------------------------------------------
rng = np.random.default_rng(3)
for name, dtype, tol in (("B", "float32", 2e-5), ("D", "bfloat16", 2e-2), ("F", "bfloat16", 2e-2)):
    cfg = tiny_configs()[name]
    with tempfile.TemporaryDirectory() as d:
        write_random_model(cfg, 5, d, scales=InitScales(matrix=0.1, embedding=1.0, head=0.1, norm=0.1))
        pc, pw = P.read_model(d)
        eng = Engine(Model.from_dir(d, dtype=dtype), max_tokens=2048)
    prompts = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in (130, 5, 70)]
    extra = [rng.integers(0, cfg.vocab_size, size=3).tolist() for _ in prompts]
    slots = [eng.new_sequence() for _ in prompts]
    got = [eng.step(list(zip(slots, prompts))).cpu().numpy()]
    for k in range(3):
        got.append(eng.step([(s, [e[k]]) for s, e in zip(slots, extra)]).cpu().numpy())
    eng.truncate(slots[0], 90)
    got.append(eng.step([(slots[0], prompts[0][90:100])]).cpu().numpy())
    worst = 0.0
    for i, (p, e) in enumerate(zip(prompts, extra)):
        ref = P.forward_logits(p + e, pc, pw)
        rows = [got[0][i]] + [got[1 + k][i] for k in range(3)]
        want = [ref[len(p) - 1]] + [ref[len(p) + k] for k in range(3)]
        worst = max(worst, max(float(np.max(np.abs(a - b)) / np.max(np.abs(ref))) for a, b in zip(rows, want)))
    ref = P.forward_logits(prompts[0][:100], pc, pw)
    worst = max(worst, float(np.max(np.abs(got[4][0] - ref[-1])) / np.max(np.abs(ref))))
    for s in slots:
        eng.end_sequence(s)
    report["clean"].append({"config": name, "dtype": dtype, "error": worst, "tolerance": tol, "status": ops.checked_status(),
                            "tc5": ops.tc5_status()})

# ---- wrong indices are caught, and the kernels run to their end -----------------------------
ints = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
table = torch.randn(50, 16, device=DEV)
out = torch.empty((3, 16), device=DEV)
ops.embed_gather(table, ints([1, 57, 2]), out)
report["caught"]["token id"] = ops.checked_status()
report["token_id_row_is_row_0"] = bool(torch.equal(out[1], table[0]))

ids = ints([0, 9, 1])
ops.gather_tokens(ids, ints([5, 6, 7]))
report["caught"]["token source"] = ops.checked_status()

heads, kvh, d, pages = 2, 1, 16, 4
bt = ints([[0, 1], [2, 3]])
k_plane, v_plane = torch.zeros((pages, kvh, 64, d), device=DEV), torch.zeros((pages, kvh, 64, d), device=DEV)
qkv = torch.randn(2, (heads + 2 * kvh) * d, device=DEV)
cos, sin = torch.ones((256, d // 2), device=DEV), torch.zeros((256, d // 2), device=DEV)
args = lambda pos, slot, tbl: (qkv.clone(), heads, kvh, d, None, None, 0.0, cos, sin, d, ints(pos), ints([0, 1]), ints(slot), tbl, k_plane, v_plane, True)
ops.qk_norm_rope_kv_write(*args([3, 130], [0, 1], bt))          # position 130 needs a third page of a two-page row
report["caught"]["logical page"] = ops.checked_status()
ops.qk_norm_rope_kv_write(*args([3, 5], [0, 7], bt))            # slot 7 of a table of two
report["caught"]["slot"] = ops.checked_status()
ops.qk_norm_rope_kv_write(*args([3, 5], [0, 1], ints([[0, 1], [2, 9]])))   # fine: the bad entry is not reached
report["unreached_entry"] = ops.checked_status()
ops.qk_norm_rope_kv_write(*args([3, 70], [0, 1], ints([[0, 1], [2, 9]])))  # page 9 of a plane of four
report["caught"]["physical page"] = ops.checked_status()
ops.qk_norm_rope_kv_write(*args([3, 70], [0, 1], bt)[:7] + (cos[:40], sin[:40]) + args([3, 70], [0, 1], bt)[9:])  # position 70, tables of 40
report["caught"]["rope position"] = ops.checked_status()

q = torch.randn(1, heads * d, device=DEV)
o = torch.empty_like(q)
ops.attention(q, o, k_plane, v_plane, ints([[0, 11]]), ints([0]), ints([0]), ints([1]), ints([100]), 1, 1, heads, kvh, d, 0.25)
report["caught"]["attention page"] = ops.checked_status()
report["attention_finite"] = bool(torch.isfinite(o).all())

tbl = torch.zeros((2, 2), dtype=torch.int32, device=DEV)
ops.block_table_set(tbl, ints([5, 0, 1, 1, 1, 3]), 2)
report["caught"]["triple"] = ops.checked_status()
report["table_after"] = tbl.cpu().tolist()
torch.cuda.synchronize()
print("REPORT " + json.dumps(report))
'''


def test_the_checked_build_trips_nothing_on_the_engines_own_steps_and_catches_wrong_indices():
    env = dict(os.environ, GOPHONIC_B200_CHECKED="1")
    proc = subprocess.run([sys.executable, "-c", SCRIPT], cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    line = next(l for l in proc.stdout.splitlines() if l.startswith("REPORT "))
    r = json.loads(line[len("REPORT "):])
    assert r["checked"]
    for run in r["clean"]:
        assert run["status"] is None and run["tc5"] == 0, run
        assert run["error"] < run["tolerance"], run
    caught = r["caught"]
    where, what, value, bound, count = caught["token id"]
    # every thread that meets the index counts it
    assert (where, value, bound) == ("rows", 57, 50) and count >= 1 and "token id" in what and r["token_id_row_is_row_0"]
    assert caught["token source"][2:4] == [9, 3]
    assert caught["logical page"][1].startswith("a position beyond the pages") and caught["logical page"][2:4] == [2, 2]
    assert caught["slot"][2:4] == [7, 2] and "slot" in caught["slot"][1]
    assert r["unreached_entry"] is None
    assert caught["physical page"][2:4] == [9, 4]
    assert caught["rope position"][2:4] == [70, 40]
    assert caught["attention page"][0].startswith("attention") and caught["attention page"][2:4] == [11, 4] and r["attention_finite"]
    assert caught["triple"][2:4] == [5, 2] and r["table_after"] == [[0, 0], [0, 3]]


def test_the_ordinary_build_carries_no_checks():
    from gophonic_b200 import ops
    if os.environ.get("GOPHONIC_B200_CHECKED", "") in ("", "0"):
        assert not ops.is_checked_build() and ops.checked_status() is None
