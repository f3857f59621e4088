"""Process-group cache (reference: src/etha/pg_utils.py:1-19).

`dist.new_group` is collective over the whole world, so callers that do use sub-groups must create
them in the same order everywhere; the cache keys on the sorted rank tuple.  The executors of this
package need no sub-groups; the cache serves user code and the DTensor-based comparison methods.
"""

import torch.distributed as dist

_PROCESS_GROUP_CACHE: dict[tuple[int, ...], "dist.ProcessGroup"] = {}


def get_or_create_process_group(ranks: list[int]):
    key = tuple(sorted(int(r) for r in ranks))
    group = _PROCESS_GROUP_CACHE.get(key)
    if group is None:
        group = dist.new_group(ranks=list(key))
        _PROCESS_GROUP_CACHE[key] = group
    return group


def clear_process_group_cache() -> None:
    _PROCESS_GROUP_CACHE.clear()
