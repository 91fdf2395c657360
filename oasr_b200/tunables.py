"""Process-wide integer tunables of the native library (tile shapes etc.).

``gemm_bn``: 0 lets the heuristic choose the GEMM tile width, 64 / 128 / 256 force it.
``lsm_path``: the CTC head - 0 (default) chooses by size, 1 the fused two-sweep kernel, 2 an fp32 logits GEMM followed by
an in-place row log-softmax kernel (fp32 output only).
``gemm_pairs``: 1 runs large dense GEMMs on CTA pairs (tcgen05 cta_group::2), 0 (default) on single-CTA tiles.
``dwconv_path``: 2 (default) runs the depthwise conv of kernel size 9 / 15 on the rolling register-window kernel (other sizes
up to 15 on the run-at-once register-streaming kernel), 0 all of them on the run-at-once kernel, 1 on the shared-memory tiled one.
``fmha_chunk_path``: 1 (default) runs paged rel-pos attention with <= 16 query frames on the warp-per-(stream, head)
kernel, 0 always on the 128-row tcgen05 kernel.
``fmha_relpos_path``: 1 (default) runs packed relative-position attention on the two-CTAs-per-SM kernel, 0 on the general one.
``conv1_mma``: 1 (default) runs the first subsampling convolution (parity-split output, 256 / 512 channels) as a K = 32
split-bf16 GEMM on the tensor cores, 0 as the fp32 stencil kernel.
``conv2_pairs``: 1 (default) runs the second subsampling convolution on CTA pairs over all output channels (widths
128 / 256 / 512), 0 on the single-CTA implicit-GEMM kernel.
``fused_addnorm``: 1 (default) runs the last Linear of every Conformer sub-layer fused with the residual add and the
following norm (widths 128 / 256 / 512) when the batch's 256-row tiles fill the GPU, 2 whenever the width allows it, 0
always as gemm + add_norm_f32.
``qkv_dup``: 1 (default) computes the query block of the fused q/q/k/v projection once and stores it twice with its two
biases (widths that are multiples of 256), 0 multiplies by the duplicated weight block.
``pdl``: 1 (default) launches the hot kernels with programmatic stream serialisation, 0 in plain stream order.
"""
from __future__ import annotations

from . import _lib


def set(name: str, value: int) -> None:  # noqa: A001 - mirrors the C entry point's name
    _lib.call("oasr_b200_set_tunable", name.encode(), int(value))
