"""CPU oracle for the paged KV-cache hot path: TEST INFRASTRUCTURE ONLY.

`kv_oracle` restates the reference's bookkeeping crate in Python; `c_oracle` binds the C
restatement of the kernel math (`kriya_oracle.c`).  Nothing under `kriya_rt_b200/` imports this
package; only `tests/`, the smoke check and the benchmark's CPU-baseline leg do.
"""
