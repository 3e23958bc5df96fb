"""Placement of work on the GPUs of one node (no data-path collective except the long-context merge).

* batch / kv-head sharding (decode, verify, prefill): every GPU owns whole sequences or whole kv
  heads; results are independent (the reference shards attention by kv head across its TP ranks,
  crates/warp34-host/src/model/forward.rs:1085-1086).
* page sharding of one long sequence: rank r holds a contiguous, page-aligned token range; each
  rank runs warp34_paged_attention_partial_f16 over its range and the (acc, m, l) triples are
  all-gathered and merged (warp34_paged_attention_merge_shards_f16).
"""
PAGE = 16


def split_batch(num_items, world, rank):
    """Contiguous share [lo, hi) of num_items for `rank`; sizes differ by at most one."""
    base, rem = divmod(num_items, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def split_kv_heads(num_kv_heads, num_q_heads, world, rank):
    """(kv head range, q head range) of `rank` when kv heads divide over `world` ranks; q heads
    follow their kv head.  world may exceed num_kv_heads only by a factor that then splits the
    batch instead (returns the batch split factor as third value)."""
    if world <= num_kv_heads:
        assert num_kv_heads % world == 0
        per = num_kv_heads // world
        g = num_q_heads // num_kv_heads
        return (rank * per, (rank + 1) * per), (rank * per * g, (rank + 1) * per * g), 1
    assert world % num_kv_heads == 0
    batch_split = world // num_kv_heads
    h = rank // batch_split
    g = num_q_heads // num_kv_heads
    return (h, h + 1), (h * g, (h + 1) * g), batch_split


def split_pages(num_tokens, world, rank):
    """Token range [lo, hi) of `rank` for a sequence of num_tokens, cut at page boundaries and as
    even as pages allow; trailing ranks may be empty for short sequences."""
    pages = (num_tokens + PAGE - 1) // PAGE
    p_lo, p_hi = split_batch(pages, world, rank)
    return min(p_lo * PAGE, num_tokens), min(p_hi * PAGE, num_tokens)
