"""The header of a safetensors file, read by the tests' own few lines."""
import json
import struct


def names_and_shapes(path):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n).decode("utf-8"))
    return {k: v["shape"] for k, v in header.items() if k != "__metadata__"}
