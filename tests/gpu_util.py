"""Helpers shared by the GPU parity tests: device buffers through torch, the executor through the C ABI."""
import numpy as np
import torch

from kriya_rt_b200.executor import CudaExecutor
from oracle import c_oracle as O


def dev16(a: np.ndarray) -> torch.Tensor:
    """uint16 bit patterns -> int16 device tensor (same bits)."""
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).cuda()


def host16(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy().view(np.uint16)


def make_executor(shape, num_blocks, num_layers=1, **kw) -> CudaExecutor:
    return CudaExecutor(num_layers=num_layers, num_kv_blocks=num_blocks, block_size_tokens=shape.block_size,
                        num_q_heads=shape.num_q_heads, num_kv_heads=shape.num_kv_heads, head_dim=shape.head_dim,
                        dtype=shape.dtype, rope_theta=shape.rope_theta, **kw)


def fill_cache(ex: CudaExecutor, layer: int, cache_k: np.ndarray, cache_v: np.ndarray) -> None:
    k, v = ex.layer_cache_views(layer)
    k.copy_(dev16(cache_k))
    v.copy_(dev16(cache_v))
    torch.cuda.synchronize()


def read_cache(ex: CudaExecutor, layer: int):
    ex.sync()
    k, v = ex.layer_cache_views(layer)
    return host16(k), host16(v)


def oracle_gqa(ex: CudaExecutor, softcap=0.0, sm_scale=None) -> O.GqaParams:
    p = ex.gqa_params(logit_softcap=softcap, sm_scale=sm_scale)
    return O.GqaParams(p.num_q_heads, p.num_kv_heads, p.head_dim, p.block_size_tokens, p.max_split_k_tiles,
                       p.max_query_tokens, p.sm_scale, p.logit_softcap)


def oracle_rope(p) -> O.RopeParams:
    return O.RopeParams(p.num_q_heads, p.num_kv_heads, p.head_dim, p.rotary_dim, p.block_size_tokens, p.apply_qk_norm,
                        p.rms_eps, p.rope_theta, p.max_seq_len, p.has_table, 0, 0)


TOL = {0: 1e-2, 1: 2e-3}  # max-abs vs the fp32 oracle: bf16, fp16
