"""Token sampling for the generation engine.

The fast path (temperature only, the setting the RL recipes use) is one kernel per step:
Gumbel-max over the logits row, which is an exact draw from ``softmax(z / T)``, fused with the
log-probability of the drawn token (``csrc/decode.cu``).  top-k / top-p / min-p go through a
PyTorch path that masks the logits first.  Mirrors the sampling parameters the reference forwards
to its engine (skyrl/backends/skyrl_train/inference_servers/engine_utils.py:55-82).
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib

_cfg_done = False


def _k():
    global _cfg_done
    lib = _lib.kernels()
    if not _cfg_done:
        vp, ci, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        lib.sb_sample_gumbel.argtypes = [vp, ci, cl, ci, ci, vp, ctypes.c_ulonglong, vp, vp, vp, vp]
        lib.sb_embed_gather.argtypes = [vp, vp, vp, ci, ci, vp]
        _cfg_done = True
    return lib


def mask_logits(logits: torch.Tensor, top_k: int = -1, top_p: float = 1.0, min_p: float = 0.0) -> torch.Tensor:
    """Return fp32 logits with everything outside the top-k / nucleus / min-p set at -inf."""
    z = logits.float()
    if top_k is not None and 0 < top_k < z.shape[-1]:
        kth = torch.topk(z, top_k, dim=-1).values[..., -1:]
        z = z.masked_fill(z < kth, float("-inf"))
    if top_p is not None and top_p < 1.0:
        sz, idx = torch.sort(z, dim=-1, descending=True)
        probs = torch.softmax(sz, dim=-1)
        cum = probs.cumsum(-1)
        remove = (cum - probs) >= top_p
        sz = sz.masked_fill(remove, float("-inf"))
        z = torch.full_like(z, float("-inf")).scatter(-1, idx, sz)
    if min_p is not None and min_p > 0.0:
        probs = torch.softmax(z, dim=-1)
        z = z.masked_fill(probs < min_p * probs.max(-1, keepdim=True).values, float("-inf"))
    return z


def sample(logits: torch.Tensor, temperature: torch.Tensor, seed: int, step_counter: torch.Tensor | None = None,
           out_tokens: torch.Tensor | None = None, out_logprobs: torch.Tensor | None = None,
           generator: torch.Generator | None = None):
    """Draw one token per row of ``logits [n, V]``; returns ``(tokens int32 [n], logprobs fp32 [n])``.

    ``temperature`` is a per-row fp32 tensor; rows with temperature <= 0 are decoded greedily.  The
    returned log-probability is that of the drawn token under ``softmax(logits / temperature)``
    (temperature 1 for greedy rows).
    """
    n, V = logits.shape
    if logits.is_cuda:
        if out_tokens is None:
            out_tokens = torch.empty(n, device=logits.device, dtype=torch.int32)
        if out_logprobs is None:
            out_logprobs = torch.empty(n, device=logits.device, dtype=torch.float32)
        assert logits.stride(1) == 1 and logits.dtype in (torch.bfloat16, torch.float32)
        code = _k().sb_sample_gumbel(logits.data_ptr(), int(logits.dtype == torch.bfloat16), logits.stride(0), n, V,
                                     temperature.data_ptr(), seed & ((1 << 64) - 1), _lib.ptr(step_counter),
                                     out_tokens.data_ptr(), out_logprobs.data_ptr(), _lib.stream_ptr())
        _lib.check(code, "sb_sample_gumbel")
        return out_tokens, out_logprobs
    t = temperature.float().clamp_min(0)
    greedy = t <= 0
    z = logits.float() / torch.where(greedy, torch.ones_like(t), t)[:, None]
    lp = torch.log_softmax(z, dim=-1)
    if generator is None:
        generator = torch.Generator().manual_seed(seed)
    u = torch.rand(z.shape, generator=generator).clamp_min(1e-20)
    gum = -torch.log(-torch.log(u))
    tok = torch.where(greedy, z.argmax(-1), (z + gum).argmax(-1))
    return tok.to(torch.int32), lp.gather(-1, tok[:, None]).squeeze(-1)


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Row gather ``table[ids]`` (no autograd; the trainer's embedding uses ``embedding`` in models)."""
    _lib.check_index("embed: token id", ids, table.shape[0])
    if not table.is_cuda:
        return table[ids.long()]
    T, H = ids.numel(), table.shape[1]
    if out is None:
        out = torch.empty((T, H), device=table.device, dtype=table.dtype)
    code = _k().sb_embed_gather(table.data_ptr(), ids.data_ptr(), out.data_ptr(), T, H, _lib.stream_ptr())
    _lib.check(code, "sb_embed_gather")
    return out
