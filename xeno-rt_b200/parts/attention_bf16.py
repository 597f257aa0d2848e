"""Choice among the bfloat16 attention kernels.  ``run`` returns False when none takes the case,
and the caller uses the kernel that takes any."""
from __future__ import annotations

from ..cache.spec import BLOCK_TOKENS
from ..csrc import ops
from .context import context_bucket

DECODE_BLOCKS_PER_SM = 3   # 70 KB of shared memory a block at head size 128
TCGEN05_MIN_NEW = 32       # prompts at least this long use the tcgen05 attention (tiles of 128 query rows)
FUSED_COMBINE_MAX = 32     # (tokens x kv heads) up to which the splits are merged inside the attention kernel (measured again with 6 splits at 8 sequences: the second kernel is still faster there)
SPLIT_OVERHEAD_TILES = 2   # what a block costs beside its tiles (query load, merge, partials), in tiles of 64 keys
CLUSTER_MAX_SPLITS = 16   # up to ops.Tuning.decode_cluster_pairs (token, kv head) pairs the kernel runs a pair's splits
#                            as one thread-block cluster that merges itself through distributed shared memory (csrc/
#                            attention_decode.cu has the same two numbers); a split then costs the merge far less
CLUSTER_MERGE_TILES = 0.2
SPLIT_MERGE_TILES = 0.6    # what every further split costs the merge of a (token, kv head), in the same unit (measured
#                            at 1, 2 and 4 sequences: 16, 8..16 and 8 splits are the fastest there, not 32, 22 and 13)


def decode_split(n_seqs: int, n_kv_heads: int, max_context: int, sms: int, mean_context: int = 0):
    """(keys a split, number of splits) for decode attention.  Blocks run in rounds of what the GPU
    holds at once; the time is about rounds x (tiles a split + a fixed cost) + a cost of merging that
    grows with the splits, so the split count is chosen to fill the last round (512 pairs of sequence
    and kv head in 2 splits are 2.3 rounds and run like 3; in 4 splits they are 4.6 rounds of half the
    length).  At least two tiles a split where the context allows.  ``sms``: the device's
    multiprocessors.  ``mean_context`` (0: all as long as the longest): what a sequence holds on
    average; a split beyond a sequence's end has no keys and ends at once, so with unequal lengths
    only mean / keys-a-split of a sequence's blocks fill the rounds, and finer splits keep the one
    long sequence from being the whole step's time."""
    blocks = max(1, (max_context + BLOCK_TOKENS - 1) // BLOCK_TOKENS)
    mean_blocks = blocks if mean_context <= 0 else min(blocks, max(1, -(-mean_context // BLOCK_TOKENS)))
    pairs = max(1, n_seqs * n_kv_heads)
    slots = sms * DECODE_BLOCKS_PER_SM
    costs = {}
    for splits in range(1, max(1, min((blocks + 1) // 2, 64)) + 1):
        tiles = -(-blocks // splits)
        real = -(-blocks // tiles)  # splits that hold keys of the longest sequence
        working = min(real, -(-mean_blocks // tiles))  # and of a sequence of mean length
        # clusters only where the lengths are about equal: a cluster holds its places until its longest
        # block is done (measured with 16 lengths between 249 and 1,997: 166 against 141 microseconds a layer)
        clustered = (pairs <= ops.tuning().decode_cluster_pairs and real <= CLUSTER_MAX_SPLITS
                     and mean_blocks == blocks)
        # whole clusters have to find room: about two blocks a multiprocessor instead of three (measured at 4
        # sequences: 8 splits, 256 blocks, beat 13 and 16)
        rounds = -(-pairs * working // (sms * 2 if clustered else slots))
        merge = CLUSTER_MERGE_TILES if clustered else SPLIT_MERGE_TILES
        costs.setdefault(real, rounds * (tiles + SPLIT_OVERHEAD_TILES) + merge * real)
    least = min(costs.values())
    # among the counts within 4 % of the least cost: one that divides the blocks evenly if there is one, then the smallest
    close = [n for n, c in costs.items() if c <= 1.04 * least]
    best = min(close, key=lambda n: (blocks % n != 0, n))
    chunk = BLOCK_TOKENS * (-(-blocks // best))
    return chunk, -(-blocks * BLOCK_TOKENS // chunk)


def visible_span(context: int, window: int) -> int:
    """Keys between the cache block that holds a token's first visible key and the token itself, at most: the
    whole context without a window (0), else the window and what is left of its first block."""
    if window <= 0:
        return context
    return min(context, -(-(window + BLOCK_TOKENS - 1) // BLOCK_TOKENS) * BLOCK_TOKENS)


def _decode_split_of(ctx, n_kv_heads: int, device, window: int = 0):
    """(keys a split, splits, whether splits may merge as clusters) for the step's lengths, by their powers of
    two.  The kernels count a windowed layer's splits from the block of the first visible key, so its splits
    are cut from the window's span however long the sequences are."""
    sms = ops.device_state(device)[2]
    longest = visible_span(context_bucket(ctx.max_context), window)
    mean = min(longest, visible_span(context_bucket(ctx.mean_context), window)) if ctx.mean_context > 0 else 0
    return decode_split(ctx.n_tokens, n_kv_heads, longest, sms, mean) + (mean == 0 or mean == longest,)


def decode_from_qkv(out, qkv, k_offset, v_offset, q_norm, k_norm, eps, cos_sin, pairing, ctx, store, n_heads, n_kv_heads,
                    head_dim, scale, window, write_kv) -> bool:
    """A decode step's attention straight from the q/k/v product's output: the kernel does the head norms,
    the rotation and the cache write itself (one kernel and one boundary less a layer).  False where that
    kernel does not take the case; the caller then runs the rotation kernel and ``run``."""
    rope_half = 0 if cos_sin is None else cos_sin.shape[1]
    if not (ctx.all_single and ctx.n_tokens <= 65535
            and ops.attention_decode_takes_qkv(n_heads, n_kv_heads, head_dim, rope_half, pairing)):
        return False
    chunk, n_splits, clusters = _decode_split_of(ctx, n_kv_heads, qkv.device, window)
    fused = ctx.n_tokens * n_kv_heads <= FUSED_COMBINE_MAX
    ops.attention_decode_qkv(out, qkv, k_offset, v_offset, q_norm, k_norm, eps, cos_sin, store.k, store.v, ctx.tok_slot,
                             ctx.tok_pos, store.block_table, n_heads, n_kv_heads, head_dim, scale, window, chunk, n_splits,
                             write_kv=write_kv, fused=fused, clusters=clusters)
    return True


def run(out, q, ctx, store, n_heads, n_kv_heads, head_dim, scale, window) -> bool:
    if n_heads // n_kv_heads > 16:
        return False
    if ctx.all_single and ctx.n_tokens <= 65535:
        chunk, n_splits, clusters = _decode_split_of(ctx, n_kv_heads, q.device, window)
        # few sequences: the last block of a (token, kv head) merges its splits (one launch less);
        # many: a second kernel merges them with more threads (measured faster from 8 sequences on)
        fused = ctx.n_tokens * n_kv_heads <= FUSED_COMBINE_MAX
        ops.attention_decode(out, q, store.k, store.v, ctx.tok_slot, ctx.tok_pos, store.block_table, n_heads,
                             n_kv_heads, head_dim, scale, window, chunk, n_splits, fused=fused, clusters=clusters)
        return True
    if ctx.n_seqs <= 65535 and n_heads <= 65535:
        if (head_dim == 128 and window == 0 and ctx.max_new >= TCGEN05_MIN_NEW
                and ops.tuning().prefill_attention != "mma"):
            ops.attention_prefill_tcgen05(out, q, store.k, store.v, ctx.cu_seqlens, ctx.seq_slot, ctx.seq_start,
                                          store.block_table, ctx.max_new, n_heads, n_kv_heads, head_dim, scale)
            return True
        ops.attention_prefill(out, q, store.k, store.v, ctx.cu_seqlens, ctx.seq_slot, ctx.seq_start,
                              store.block_table, ctx.max_new, n_heads, n_kv_heads, head_dim, scale, window)
        return True
    return False
