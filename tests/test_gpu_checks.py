"""The checks build of the kernels (``kernels.enable_checks()``): page ids, cache slots and token ids that a kernel
reads from memory are compared with limits; a value out of range is recorded and replaced by a safe one.  It runs
in a process of its own, because the switch is a compile-time one and this process has its libraries loaded."""

import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent

SCRIPT = r'''
import json, sys, tempfile
sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + "/tests")
import torch
from inf_engine_b200 import kernels
kernels.enable_checks()
from inf_engine_b200 import Engine, Request
from inf_engine_b200.config import parse_config_dict
from inf_engine_b200.weights import write_random_model
from helpers import TINY_F

with tempfile.TemporaryDirectory() as tmp:
    write_random_model(parse_config_dict(TINY_F), 5, tmp, std=0.05)
    engine = Engine.from_dir(tmp, dtype="bfloat16", n_total_blocks=40, block_size=16, max_tokens_per_step=256)
long_prompt = [(7 * i + 3) % 1000 for i in range(150)]
out = engine.run_offline([Request(0, long_prompt, 4), Request(1, [11, 400, 23], 4)])   # raises if a check had failed
result = {{"clean": kernels.read_check_words(), "generated": [len(out[0]), len(out[1])]}}

# Now the checker is told that the pool has 3 pages and 48 slots and the vocabulary 10 tokens: pages, slots and
# tokens that are perfectly valid trip it, and the kernels leave them alone (no page, no slot), so nothing is
# read or written out of bounds whatever the check does.
kernels.set_check_limits(3, 48, 10)
engine.completed.clear()
engine.submit(Request(2, long_prompt, 3))
engine.submit(Request(3, [5, 6, 7, 8], 3))
while engine.has_work:
    engine.step()
torch.cuda.synchronize()
try:
    kernels.check_device_errors()
    result["raised"] = None
except kernels.KernelError as e:
    result["raised"] = str(e)
kernels.set_check_limits(40, 40 * 16, 1000)
engine.completed.clear()
again = engine.run_offline([Request(4, long_prompt, 4)])
result["after"] = kernels.read_check_words()
result["same_tokens"] = again[4] == out[0]
print("RESULT " + json.dumps(result))
'''


@pytest.mark.gpu
def test_a_checks_build_records_values_out_of_range_and_uses_none_of_them():
    r = subprocess.run([sys.executable, "-c", SCRIPT.format(root=str(ROOT))], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    line = [x for x in r.stdout.splitlines() if x.startswith("RESULT ")][-1]
    res = json.loads(line[len("RESULT "):])
    assert res["clean"] == [] and res["generated"] == [4, 4]          # an ordinary run trips nothing
    msg = res["raised"]
    assert msg and "checks build" in msg
    # the prompt's token ids and slots (embedding, rotation and cache write), the page ids in the prompt portion's
    # attention and in the decode attention
    assert "elementwise" in msg and "attention_tcgen05" in msg and "attention_mma" in msg
    assert "page id" in msg and ("token id" in msg or "cache slot" in msg)
    # the words were cleared by the read, and with the true limits back the engine generates what it generated before
    assert res["after"] == [] and res["same_tokens"]
