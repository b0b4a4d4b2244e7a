"""Micro-batch splitting of call arguments (behaviour of pfeife/batch.py:30-132).

Every tensor leaf is split on dim 0 into ``n`` chunks with ``torch.tensor_split``, python lists
are cut into ``n`` consecutive slices, every other leaf is replicated.
"""
from __future__ import annotations

from typing import Any, Dict, List, Sequence, Tuple

import torch
from torch.utils._pytree import tree_flatten, tree_unflatten


def _is_leaf(v: Any) -> bool:
    # a list of non-containers is chunked as a whole instead of being flattened
    return isinstance(v, list) and all(not isinstance(e, (list, tuple, dict)) for e in v) \
        and not any(torch.is_tensor(e) for e in v)


def _chunks_of(v: Any, n: int) -> Sequence[Any]:
    if torch.is_tensor(v):
        if v.dim() == 0:
            return [v] * n
        return torch.tensor_split(v, n, 0)
    if isinstance(v, list):
        size = (len(v) + n - 1) // n
        return [v[i * size:(i + 1) * size] for i in range(n)]
    return [v] * n


def split_tree(tree: Any, n: int) -> List[Any]:
    flat, spec = tree_flatten(tree, is_leaf=_is_leaf)
    per_leaf = [_chunks_of(v, n) for v in flat]
    return [tree_unflatten([c[i] for c in per_leaf], spec) for i in range(n)]


def shard_dict_of_args(args_dict: Dict[Any, Any], batch_split: int) -> List[Dict[Any, Any]]:
    keys = list(args_dict.keys())
    per_key = {k: split_tree(args_dict[k], batch_split) for k in keys}
    return [{k: per_key[k][i] for k in keys} for i in range(batch_split)]


def split_args_kwargs(args: Tuple[Any, ...], kwargs: Dict[str, Any], batch_split: int
                      ) -> Tuple[List[Tuple[Any, ...]], List[Dict[str, Any]]]:
    """-> (list of per-micro-batch args tuples, list of per-micro-batch kwargs dicts)."""
    kwargs = kwargs or {}
    k = shard_dict_of_args(kwargs, batch_split)
    if args is None:      # as in the reference: a call without positional arguments
        return [(None,) for _ in range(batch_split)], k
    a = shard_dict_of_args(dict(enumerate(args)), batch_split)
    args_split = [tuple(chunk[i] for i in range(len(args))) for chunk in a]
    return args_split, k


def send_value(value: Any, device) -> Any:
    from . import to_device
    return to_device(value, device)
