"""Optional Ray import.  Ray is not required: without it, rollout workers are
in-process objects behind the same handles (reference: ``vrl/distributed/ray/dependencies.py``)."""

from __future__ import annotations

import os
import socket
from typing import Any


def ray_available() -> bool:
    try:
        import ray  # noqa: F401

        return True
    except Exception:  # noqa: BLE001
        return False


def require_ray() -> Any:
    try:
        import ray

        return ray
    except Exception as exc:  # noqa: BLE001
        raise ImportError("ray is not installed; the in-process worker path needs no Ray") from exc


def current_node_ip() -> str:
    if ray_available():
        try:
            import ray

            return ray.util.get_node_ip_address()
        except Exception:  # noqa: BLE001
            pass
    try:
        return socket.gethostbyname(socket.gethostname())
    except OSError:
        return "127.0.0.1"


def current_gpu_ids() -> list[int]:
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    if visible:
        return [int(x) for x in visible.split(",") if x.strip().lstrip("-").isdigit()]
    try:
        import torch

        return list(range(torch.cuda.device_count()))
    except Exception:  # noqa: BLE001
        return []
