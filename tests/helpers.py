"""Helpers shared by the parity tests."""

import hashlib
from typing import List

import numpy as np
import torch


def digest_tensor(t) -> str:
    t = t.get_raw() if hasattr(t, "get_raw") else t
    raw = t.detach().contiguous().reshape(-1).view(torch.uint8).cpu().numpy().tobytes()
    return hashlib.sha256(raw).hexdigest()[:16]


def record(t) -> List:
    """[shape, dtype, digest] in the form tests/golden/reference_outputs.json stores."""
    t = t.get_raw() if hasattr(t, "get_raw") else t
    return [list(t.shape), str(t.dtype).replace("torch.", ""), digest_tensor(t)]


def digest_bytes(raw: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(raw).tobytes()).hexdigest()[:16]


def tensor_bytes(t) -> np.ndarray:
    t = t.get_raw() if hasattr(t, "get_raw") else t
    return t.detach().contiguous().reshape(-1).view(torch.uint8).cpu().numpy()


def free_port() -> int:
    """A TCP port that is free on 127.0.0.1 right now, for a test's process-group rendezvous."""
    import socket

    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def rendezvous(out_dir: str, token) -> str:
    """``init_method`` for a test's process group: a file in the test's own directory.  No TCP
    port is involved, so two tests (or two test runs on one machine) cannot collide on one."""
    import os

    return "file://" + os.path.join(str(out_dir), f"rendezvous_{token}")
