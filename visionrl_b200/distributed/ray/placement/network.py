"""Stable ordering key for worker placement: IPv4 octets, then GPU id, then index
(reference: ``vrl/distributed/ray/placement/network.py:8-25``)."""

from __future__ import annotations


def ip_sort_key(ip: str) -> tuple:
    parts = ip.split(".")
    if len(parts) == 4 and all(p.isdigit() for p in parts):
        return (0, *(int(p) for p in parts))
    return (1, ip)


def bundle_sort_key(ip: str, gpu_id: int | None, index: int) -> tuple:
    return (ip_sort_key(ip), -1 if gpu_id is None else int(gpu_id), int(index))


def sort_node_gpu_key(item: tuple) -> tuple:
    """The same ordering for an ``(index, node, gpu_id)`` triple, the form placement code sorts."""
    index, node, gpu_id = item
    return bundle_sort_key(str(node), None if gpu_id is None or int(gpu_id) < 0 else int(gpu_id), int(index))
