"""Choice of a quality level per chunk under a bandwidth trace and a latency target.

Mirrors config_selection of the reference (src/utils.py:294-314), which reads one stored blob per
(chunk, QUANT_LEVEL) and keeps, for every chunk, the highest level whose transfer time fits the
chunk's share of the target.  Here the blob sizes are passed in (they come from
CacheGenSerializer.encode_levels), nothing is read from disk.
"""
from typing import Dict, List, Sequence, Tuple


def level_sizes(encoded_levels: Sequence, levels: Sequence[int] = (1, 2, 3)) -> Dict[int, int]:
    """{level: size in bytes of the pickled blob} for one chunk's encode_levels result."""
    return {lv: len(eo.to_bytes()) for lv, eo in zip(levels, encoded_levels)}


def config_selection(all_bws: Sequence[float], chunk_delay: float, slo: float,
                     sizes: Sequence[Dict[int, int]]) -> Tuple[float, List[int]]:
    """all_bws[i]: bandwidth in Gbit/s while chunk i is sent; sizes[i][level]: blob bytes of chunk i at
    that level; slo: target for the whole context in seconds, split evenly over the chunks;
    chunk_delay: what a chunk costs when no level fits and it is recomputed from text (level 0).
    Returns (time to first token, level per chunk); levels are tried from the highest down."""
    num_chunks = len(sizes)
    ttft, configs = 0.0, []
    for chunk_id, by_level in enumerate(sizes):
        bw = all_bws[chunk_id]
        for level in sorted(by_level, reverse=True):
            seconds = by_level[level] / 1e9 * 8 / bw
            if seconds < slo / num_chunks:
                ttft += seconds
                configs.append(level)
                break
        else:
            ttft += chunk_delay
            configs.append(0)
    return ttft, configs
