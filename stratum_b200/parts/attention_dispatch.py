"""Which attention kernel serves a given step.

float32, and head sizes the tensor-core kernel refuses (above 128, or no multiple of 16): the CUDA-core
kernel with the fixed key order.  bfloat16 decode steps: the TMA-fed kernel that spreads all pages evenly over
the SMs (head size 64 or 128, up to 8 heads per kv head), else the kernel whose keys are cut into splits per
sequence, which needs scratch for the partial results.  bfloat16 prompts: the tcgen05 kernel, else the tile kernel.
"""
from __future__ import annotations

import os

import torch

from .. import kernels as K
from ..cache.pages import PAGE_TOKENS

# work items (warps) wanted in flight on decode steps: 148 SMs times the warps an SM holds of the decode kernel
TARGET_WARPS = int(os.environ.get("STRATUM_ATTENTION_WARPS", 148 * 8))


MAX_SPLITS = 256                # what the merge kernel takes


def plan_splits(n_items: int, max_len: int):
    """(n_splits, keys per split) for decode steps: enough splits to fill the GPU, whole pages per split."""
    pages = max(1, (max_len + PAGE_TOKENS - 1) // PAGE_TOKENS)
    want = max(1, min(pages, MAX_SPLITS, (TARGET_WARPS + n_items - 1) // n_items))
    chunk = ((pages + want - 1) // want) * PAGE_TOKENS
    return (max_len + chunk - 1) // chunk, chunk


WHOLE_PAGES_MIN = 1184          # pages of all sequences and kv heads: eight to an SM of 148


def _stream_form() -> str:
    """STRATUM_ATTENTION_STREAM_FORM=0: never whole pages per warp (for measurements)."""
    return os.environ.get("STRATUM_ATTENTION_STREAM_FORM", "")


def run(att, qkv: torch.Tensor, cache, step, out: torch.Tensor) -> None:
    hd = att.head_dim
    if qkv.dtype != torch.bfloat16 or hd % 16 != 0 or hd > 128 or qkv.stride(0) % 8 != 0:
        K.attention_simple(qkv, cache.k, cache.v, step.token_pos, step.token_seq, cache.block_table, out,
                           att.n_heads, att.n_kv_heads, hd, PAGE_TOKENS, att.window, att.scale)
        return
    gs = att.n_heads // att.n_kv_heads
    rows_per_token = min(gs, 16)
    head_groups = (gs + 15) // 16
    if (step.all_single and hd in (64, 128) and gs <= 8 and step.n_tokens <= 1024
            and os.environ.get("STRATUM_ATTENTION_STREAM", "1") != "0"):
        # decode steps: the pages of all sequences spread evenly over the SMs, streamed by TMA.  With more than
        # two sequences the kernels after it get a head start while the last pages stream in (3 % of a step on
        # the Llama-8B shape at 8 sequences); with one or two it costs more than it gives (measured)
        # heads of 64: whole pages per warp where an SM gets more than a few pages (by the step's longest sequence;
        # measured: 93 against 119 us at 64 sequences of 4,096 tokens, 11.2 against 9.9 us at one)
        pages = step.n_tokens * att.n_kv_heads * ((step.max_len + PAGE_TOKENS - 1) // PAGE_TOKENS)
        K.attention_stream(qkv, cache.k, cache.v, step.token_pos, step.token_seq, cache.block_table, out,
                           att.n_heads, att.n_kv_heads, hd, PAGE_TOKENS, att.window, att.scale,
                           late_trigger=step.n_tokens > 2,
                           whole_pages=hd == 64 and pages >= WHOLE_PAGES_MIN and _stream_form() != "0")
    elif step.all_single:
        n_splits, chunk = plan_splits(step.n_tokens * att.n_kv_heads * head_groups, step.max_len)
        part_o = part_ml = None
        if n_splits > 1:
            n = step.n_tokens * att.n_heads * n_splits
            part_o = att.runtime.scratch("attention_part_o", n * hd, torch.float32)
            part_ml = att.runtime.scratch("attention_part_ml", n * 2, torch.float32)
        K.attention_mma(qkv, cache.k, cache.v, step.token_pos, step.token_seq, cache.block_table, None, 1, out,
                        part_o, part_ml, att.n_heads, att.n_kv_heads, hd, PAGE_TOKENS, att.window, att.scale,
                        n_splits, chunk)
    elif hd in (64, 128) and 128 % gs == 0 and os.environ.get("STRATUM_ATTENTION_TC", "1") != "0":
        # prompts: the tcgen05 kernel; a CTA owns 256 query rows (2 x 128 / gs tokens) whose two halves share every
        # key and value tile (STRATUM_ATTENTION_HALVES=1: 128 rows per CTA, two CTAs per SM; measurements)
        halves = int(os.environ.get("STRATUM_ATTENTION_HALVES", "2"))
        K.attention_tc(qkv, cache.k, cache.v, step.token_pos, cache.block_table,
                       step.query_blocks(halves * (128 // gs)), out, att.n_heads, att.n_kv_heads, hd, PAGE_TOKENS,
                       att.window, att.scale, halves)
    else:
        per_warp = 16 // rows_per_token
        K.attention_tile(qkv, cache.k, cache.v, step.token_pos, step.token_seq, cache.block_table,
                         step.query_blocks(4 * per_warp), per_warp, out, att.n_heads, att.n_kv_heads, hd,
                         PAGE_TOKENS, att.window, att.scale)


# CTAs wanted on decode steps of the general attention: two to an SM of 148.  Measured at batch 8 and 4,090 cached
# tokens, four layers (three latent, one differential): 0.166 ms with 296 against 0.209 / 0.197 / 0.191 with 148 /
# 592 / 1,184 on a 2,048-wide model, 0.288 against 0.388 / 0.344 / 0.417 on a 4,096-wide one: more ranges are more
# partial results for the finishing kernel to merge, fewer leave SMs idle.
GENERAL_TARGET_CTAS = int(os.environ.get("STRATUM_GENERAL_ATTENTION_CTAS", 148 * 2))
GENERAL_MAX_SPLITS = 64


def plan_general_splits(n_items: int, max_len: int, window: int = 0):
    """(n_splits, keys per split) for decode steps of the general attention: whole pages per split.  Ranges are
    counted from position 0 for every sequence; with a window only the last ones hold keys a row can see (the others
    leave at once), so the ranges are sized to cut the window's stretch, not the whole sequence, into enough pieces."""
    pages = max(1, (max_len + PAGE_TOKENS - 1) // PAGE_TOKENS)
    seen = pages if window <= 0 else min(pages, (window + PAGE_TOKENS - 1) // PAGE_TOKENS + 1)
    want = max(1, min(seen, GENERAL_MAX_SPLITS, (GENERAL_TARGET_CTAS + n_items - 1) // n_items))
    per = max((seen + want - 1) // want, (pages + GENERAL_MAX_SPLITS - 1) // GENERAL_MAX_SPLITS)
    chunk = per * PAGE_TOKENS
    return (max_len + chunk - 1) // chunk, chunk


def run_general_dense(att, shape, q: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, step,
                      out: torch.Tensor) -> None:
    """The tensor-core general attention of a prompt step whose sequences all begin at position 0, over keys and
    values the mixer formed for the step's tokens: plain matrices, row = packed row of the token (so sequence s's
    key of position j is row seq_start[s] + j), with 64 readable rows beyond the step's."""
    per_block = 16 // min(shape.group, 16)
    row_groups = K.attention_general_mma_row_groups(shape.v_dim)
    chunk = ((step.max_len + PAGE_TOKENS - 1) // PAGE_TOKENS) * PAGE_TOKENS
    K.attention_general_mma(shape, q, keys, values, step.token_pos, step.token_seq, None, out, PAGE_TOKENS,
                            step.query_blocks(per_block * row_groups), per_block, 1, chunk, None, None, row_groups,
                            seq_start=step.seq_start)


def run_general(att, shape, q: torch.Tensor, cache, step, out: torch.Tensor) -> None:
    """Attention of the shapes kernels.AttentionShape describes (key and value sizes of their own, values inside the
    key rows, several maps per head): q [tokens, *] holds head j's map m at column (j * maps + m) * qk_dim.
    bfloat16 with sizes in multiples of 8: the tensor-core kernel (decode steps: the keys cut into ranges that
    fill the GPU; prompts: query blocks of 16 rows); everything else: the CUDA-core kernel, float32 throughout.
    STRATUM_GENERAL_ATTENTION_MMA=0: always the CUDA-core kernel (measurements)."""
    if (not K.attention_general_mma_ok(shape, q, out, PAGE_TOKENS)
            or os.environ.get("STRATUM_GENERAL_ATTENTION_MMA", "1") == "0"):
        K.attention_general(shape, q, cache.k, cache.v, step.token_pos, step.token_seq, cache.block_table, out,
                            PAGE_TOKENS)
        return
    rows_per_token = min(shape.group, 16)
    per_block = 16 // rows_per_token
    streams = (shape.n_heads // shape.group) * ((shape.group + 15) // 16) * shape.maps
    row_groups = 1
    if step.all_single:
        qblocks = None
        n_splits, chunk = plan_general_splits(step.n_tokens * streams, step.max_len, shape.window)
    else:
        # prompts: a CTA takes several groups of 16 rows through every tile of keys, which then comes from L2 once
        row_groups = K.attention_general_mma_row_groups(shape.v_dim)
        qblocks = step.query_blocks(per_block * row_groups)
        n_splits, chunk = 1, ((step.max_len + PAGE_TOKENS - 1) // PAGE_TOKENS) * PAGE_TOKENS
    part_o = part_ml = None
    if n_splits > 1 or shape.maps > 1:
        n = step.n_tokens * shape.n_heads * shape.maps * n_splits
        part_o = att.runtime.scratch("general_attention_part_o", n * shape.v_dim, torch.float32)
        part_ml = att.runtime.scratch("general_attention_part_ml", n * 2, torch.float32)
    K.attention_general_mma(shape, q, cache.k, cache.v, step.token_pos, step.token_seq, cache.block_table, out,
                            PAGE_TOKENS, qblocks, per_block, n_splits, chunk, part_o, part_ml, row_groups)
