"""Matrix products y = x W^T.

The reference's engine uses a library for every linear layer (nn.Linear, i.e.
cuBLAS: src/dli/model/llama.py:72-74,95,190,305); so does this wrapper.  The
float32 path is true 32-bit: TF32 and reduced-precision accumulation are switched
off for the process when this module is imported, and checked at every call.
"""

from __future__ import annotations

import torch

from . import ops
from .attention import sm_count

torch.backends.cuda.matmul.allow_tf32 = False
torch.backends.cudnn.allow_tf32 = False
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False


# Up to this many tokens a layer's bfloat16 products go to the engine's own tcgen05 kernel, which
# there beats the library on three of the four shapes and fuses the next elementwise step;
# measured on B200 at Llama-3.2-1B sizes, the library's kernels win from about 12 tokens on.
# The head's product (float32 logits straight from the accumulator) stays with it up to 64.
SKINNY_MAX_TOKENS = 8
SKINNY_MAX_TOKENS_HEAD = 64


def decode_product(x: torch.Tensor, max_tokens: int = SKINNY_MAX_TOKENS) -> bool:
    """Whether a product with these activations goes to the engine's own decode kernel."""
    return x.dtype == torch.bfloat16 and x.shape[0] <= max_tokens and ops.skinny_gemm_supported(x.shape[0], x.shape[1])


# Up to this many tokens the decode product also finishes the next elementwise step (rotary and
# cache write, SiLU * up) in its epilogue; with more tokens per CTA the separate kernels, which
# spread that work over the whole GPU, are faster.
FUSED_EPILOGUE_MAX_TOKENS = 8


def fused_epilogue(x: torch.Tensor) -> bool:
    return decode_product(x) and x.shape[0] <= FUSED_EPILOGUE_MAX_TOKENS


# From this many tokens two of a layer's bfloat16 products go to the engine's tcgen05 product for many tokens, which
# does the elementwise step behind the product in its epilogue.  Measured on B200 at Llama-3.2-1B sizes (us, this
# product against the library's product plus the kernel it saves; 512 / 2,048 / 8,192 tokens): gate|up with SiLU * up
# 39/38, 102/116, 383/427: always.  q|k|v with rotary and cache write 26/37, 39/37, 87/98: when its tiles fill their
# waves (2,048 tokens are 96 tiles on 74 pairs of SMs).  The plain product takes 1.00 of the library's time for gate|up
# at 2,048 tokens, 0.96-1.07 for o and down, which stay with the library: with the residual addition and the norm's
# sums in the epilogue they were slower than the library's product and the norm kernel (the epilogue read and wrote
# the float32 residual a row per thread), so that epilogue was taken out again.
DENSE_MIN_TOKENS = 512
DENSE_TILE = (256, 256)  # tokens x features of a tile, which a pair of SMs computes
WAVE_FILL_MIN = 0.8


def _dense_tiles(tokens: int, features: int) -> int:
    return -(-tokens // DENSE_TILE[0]) * -(-features // DENSE_TILE[1])


def _dense_candidate(x, features: int) -> bool:
    return x.dtype == torch.bfloat16 and x.shape[0] >= DENSE_MIN_TOKENS and ops.dense_gemm_supported(x.shape[1], features)


def dense_product(x, features: int, epilogue: str) -> bool:
    """Whether the product of these activations with a [features, K] weight, followed by ``epilogue`` ("swiglu", "act": a
    plain feed-forward's activation, or "rotary"), goes to the engine's product for many tokens."""
    if not _dense_candidate(x, features):
        return False
    tiles, pairs = _dense_tiles(x.shape[0], features), max(1, sm_count() // 2)
    if epilogue in ("swiglu", "act"):  # the activation of a feed-forward rides for nothing under the next tile's products
        return True
    if epilogue == "rotary":
        return tiles <= pairs or tiles / (-(-tiles // pairs) * pairs) >= WAVE_FILL_MIN
    raise ValueError(f"unknown epilogue {epilogue!r}")


def project(x, weight: torch.Tensor, out_dtype: torch.dtype | None = None, max_tokens: int = SKINNY_MAX_TOKENS) -> torch.Tensor:
    """y = x W^T for a step's tokens, in x's dtype or in ``out_dtype`` (float32 for logits).  x may be
    ops.ScaledRows (rows that still lack their norm's factor): those only exist for token counts that
    the decode kernel serves, which applies the factor."""
    # TMA reads the decode product's activations: rows back to back from a 16-byte boundary (a column slice of wider rows is
    # neither, and a slice of a single row, though "contiguous", may start off the boundary): those stay with the library
    if isinstance(x, ops.ScaledRows) or (decode_product(x, max_tokens) and x.is_contiguous() and x.data_ptr() % 16 == 0):
        return ops.skinny_gemm(x, weight, out_dtype or x.dtype)
    if out_dtype == torch.float32 and x.dtype != torch.float32:
        return logits_product(x, weight)
    y = linear(x, weight)
    return y if out_dtype in (None, y.dtype) else y.to(out_dtype)


def project_bias(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    """y = x W^T + b: the bias joins the float32 sums before the one rounding (the library's product with its bias
    epilogue, at every token count); without a bias it is ``project``."""
    if bias is None:
        return project(x, weight)
    return linear_bias(x, weight, bias)


def linear_bias(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    _need_device(x, "linear_bias")
    if torch.backends.cuda.matmul.allow_tf32:
        raise RuntimeError("linear_bias: TF32 was switched on; the float32 path must stay true 32-bit")
    return torch.addmm(bias, x, weight.t())


def last_product(x: torch.Tensor, weight: torch.Tensor, defer: bool):
    """The product that ends a mixer or feed-forward: x W^T, or — if the part's owner allowed it and
    the decode kernel with its fused epilogues will serve these tokens — the product left
    uncomputed for the norm behind it (parts.base.PendingProduct)."""
    if defer and fused_epilogue(x):
        from ..parts.base import PendingProduct

        return PendingProduct(x, weight)
    return project(x, weight)


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """x [n, in] times weight [out, in] transposed; float32 accumulation in both dtypes."""
    if not x.is_cuda:
        raise RuntimeError("linear: the engine has no CPU path")
    if torch.backends.cuda.matmul.allow_tf32:
        raise RuntimeError("linear: TF32 was switched on; the float32 path must stay true 32-bit")
    return torch.matmul(x, weight.t(), out=out)


def _need_device(x: torch.Tensor, what: str) -> None:
    if not x.is_cuda:
        raise RuntimeError(f"{what}: the engine has no CPU path")


HEADS_MATVEC_MAX_TOKENS = 8  # up to this many tokens a gated per-head product goes to the engine's own small kernel


def heads_product(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, gate: torch.Tensor | None = None) -> torch.Tensor:
    """out[t, a, :] = x[t, a, :] @ weight[a]: one product per head a (x [n, heads, in] and out [n, heads, features]
    may be column slices of wider rows; weight [heads, in, features] contiguous), float32 accumulation; with ``gate``
    [n, heads * features] the result is multiplied by sigmoid(gate).  The library's strided-batched product, and the
    gate kernel behind it; for a decode step's few tokens a gated product is one kernel of the engine instead (measured
    in replayed graphs at 8 tokens, 16 heads, 192 x 128: 4.6 us against 2.4 + 5.0; without a gate the library's 2.5 us
    stand)."""
    _need_device(x, "heads_product")
    if torch.backends.cuda.matmul.allow_tf32:
        raise RuntimeError("heads_product: TF32 was switched on; the float32 path must stay true 32-bit")
    n, heads, features = out.shape
    if gate is not None and n <= HEADS_MATVEC_MAX_TOKENS and ops.heads_matvec_supported(x.shape[2], features):
        ops.heads_matvec(out, x, weight, gate)
        return out
    torch.bmm(x.transpose(0, 1), weight, out=out.transpose(0, 1))
    if gate is not None:
        ops.sigmoid_gate(out.view(n, heads * features), gate)
    return out


def batched_project(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """out[b] = x[b] @ weight[b] for x [batch, n, in] and weight [batch, in, features] (several products of one shape whose
    inputs differ, in one call of the library's batched product); float32 accumulation."""
    _need_device(x, "batched_project")
    if torch.backends.cuda.matmul.allow_tf32:
        raise RuntimeError("batched_project: TF32 was switched on; the float32 path must stay true 32-bit")
    return torch.bmm(x, weight)


def logits_product(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """x [n, in] (bfloat16 or float32) times weight [out, in] transposed, the float32 sums returned as they are."""
    _need_device(x, "logits_product")
    if x.dtype == torch.float32:
        return linear(x, weight)
    return torch.mm(x, weight.t(), out_dtype=torch.float32)
