"""Regenerates tests/golden/numeric_fixtures.npz from the CPU oracle (run from the repository root).

Contents: the oracle's fp32 decode output for the SmolLM2-shaped batch-4 case (after the fused append of
one new token per row), in fp16 and bf16 storage; the RoPE'd q and the appended K rows for the same case."""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from kriya_rt_b200 import workloads as W  # noqa: E402
from oracle import c_oracle as O  # noqa: E402


def main():
    out = {}
    for dtype, tag in ((W.FP16, "fp16"), (W.BF16, "bf16")):
        shape, batch, data = W.config1(dtype=dtype)
        rp = O.RopeParams(9, 3, 64, 64, 16, 0, 1e-6, shape.rope_theta, 4096, 1, 0, 0)
        gp = O.GqaParams(9, 3, 64, 16, 16, 1, float(np.float32(1.0) / np.sqrt(np.float32(64))), 0.0)
        q, ck, cv = data["q"].copy(), data["cache_k"].copy(), data["cache_v"].copy()
        O.rope_kv_append(q, data["k"], data["v"], ck, cv, batch.page_indptr, batch.page_indices, batch.last_page_len,
                         batch.positions, rp, dtype, table=O.rope_table(4096, 64, shape.rope_theta))
        _, outf = O.decode(q, ck, cv, batch.page_indptr, batch.page_indices, batch.last_page_len, gp, dtype)
        out[f"c1_decode_f32_{tag}"] = outf
        out[f"c1_q_rope_{tag}"] = q
        rows = []
        for r in range(batch.batch):
            blk = batch.page_indices[batch.page_indptr[r + 1] - 1]
            rows.append(ck[blk, batch.last_page_len[r] - 1])
        out[f"c1_k_rows_{tag}"] = np.stack(rows)
    np.savez_compressed(Path(__file__).parent / "numeric_fixtures.npz", **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
