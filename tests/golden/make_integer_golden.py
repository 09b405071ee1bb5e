"""Writes tests/golden/integer_state_trace.json from the reference's own scheduler objects.

Needs oracle/_ref/libsglang_ref_cpu.so (oracle/build_ref.py, which needs the reference tree).
Each case runs the prompts of tests/test_integer_state_cpu.py::small_prompts through the compiled
reference (TableManager, CacheManager, RadixPrefixCache, PrefillManager, DecodeManager, Req) and
records, per scheduler step: the batch handed to the forward pass (uids, table rows, cached and
device lengths, chunk flags, write positions), which requests finished, a checksum of the page
table and the cache sizes.

    python tests/golden/make_integer_golden.py
"""
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tests import test_integer_state_cpu as T  # noqa: E402

CASES = [
    {"seed": 11, "waves": 3, "kw": dict(num_pages=110, page_size=1, max_running_req=5, max_seq_len=96, max_extend_tokens=20)},
    {"seed": 12, "waves": 4, "kw": dict(num_pages=40, page_size=4, max_running_req=4, max_seq_len=96, max_extend_tokens=32)},
    {"seed": 13, "waves": 2, "kw": dict(num_pages=30, page_size=16, max_running_req=6, max_seq_len=96, max_extend_tokens=48)},
]


def main():
    out = {"made_by": "tests/golden/make_integer_golden.py (the reference's own objects, compiled into oracle/_ref)",
           "cases": []}
    for case in CASES:
        rng = np.random.default_rng(case["seed"])
        prompts = T.small_prompts(rng, 40)
        max_new = rng.integers(1, 9, size=len(prompts)).tolist()
        tr = T.run_trace("reference", prompts, max_new, case["waves"], **case["kw"])
        out["cases"].append({**case, "trace": json.loads(json.dumps(T._golden_record(tr)))})
        print(case["kw"], len(tr), "steps; evictable sizes seen:", sorted({s["sizes"]["evictable"] for s in tr})[:6])
    T.GOLDEN.write_text(json.dumps(out, separators=(",", ":")))
    print("wrote", T.GOLDEN, T.GOLDEN.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
