"""Offline re-writer: copy a ``.safetensors`` file so that its data section starts on a 16-byte
boundary (the job of upstream's ``examples/fix_alignment.py``).

With this loader a misaligned header costs one realign-kernel launch per 4 MiB window at load
time, so re-writing is optional; it removes the device staging ring and those launches.  The
header's JSON is kept as it is and padded with spaces, which the format allows; tensor bytes are
copied unchanged.

    python -m fastsafetensors_b200.fix_alignment in.safetensors out.safetensors
"""

from __future__ import annotations

import os
import shutil
import sys

ALIGN = 16


def aligned_copy(src: str, dst: str, align: int = ALIGN) -> bool:
    """Write ``dst`` with an aligned data section.  Returns False (and writes nothing) when
    ``src`` is aligned already."""
    size = os.path.getsize(src)
    with open(src, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise Exception(f"{src}: HeaderTooSmall, buffer_len={size}")
        n = int.from_bytes(head, "little")
        if n > size - 8:
            raise Exception(f"{src}: InvalidHeaderLength, n={n}, buffer_len={size}")
        if (8 + n) % align == 0:
            return False
        body = f.read(n)
        pad = (-(8 + n)) % align
        with open(dst, "xb") as out:
            out.write((n + pad).to_bytes(8, "little"))
            out.write(body + b" " * pad)
            shutil.copyfileobj(f, out, 16 << 20)
    return True


if __name__ == "__main__":
    if len(sys.argv) != 3:
        sys.exit(__doc__)
    changed = aligned_copy(sys.argv[1], sys.argv[2])
    print("written" if changed else "no fix is required")
