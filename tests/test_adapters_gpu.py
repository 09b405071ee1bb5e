"""The reference's own Engine, linked with the adapters of sglang.cpp_b200/adapters in place of its
four FlashInfer-bound translation units, against b200_engine_step on the same weights.

sglang.cpp_b200/adapters/build.py compiles the reference's unchanged sources from the reference
tree together with the adapters and engine_probe.cc; the link leaves no undefined symbol.  The
probe runs a prefill batch and six decode steps of two requests through sglang::Engine::forward_batch
(src/engine/engine.cc:495-544: cuBLAS linears through LibTorch, everything else through the
adapters and the C ABI) and through b200_engine_step, greedy, and prints both token sequences.
In the "qwen3-graph" case the reference's GraphRunner captures decode graphs through the backend adapter's
init_capture_graph / prepare_for_capture / prepare_for_replay and the decode steps replay them.
They must be identical: weights are N(0, 0.02) with norm weights 1, top-2 logit margins are far
above bf16 noise for a 2-layer model.
"""
import json
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
PROBE = Path(__file__).resolve().parent.parent / "sglang.cpp_b200" / "adapters" / "build" / "engine_probe"


@pytest.mark.skipif(not PROBE.exists(), reason="the probe was not built (needs the reference tree at build time)")
@pytest.mark.parametrize("model", ["qwen3", "llama", "qwen3-graph"])
def test_reference_engine_on_the_adapters_gives_the_step_runners_tokens(model):
    res = subprocess.run([str(PROBE), model], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-3000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("{")][-1]
    out = json.loads(line)
    ref, own = out["reference_engine_with_adapters"], out["b200_engine_step"]
    assert len(ref) == len(own) == 14      # (1 prefill + 6 decode steps) x 2 requests
    assert ref == own, f"{model}: {ref} vs {own}"
