"""Portable synthetic operands for the large golden cases: a fixed integer hash of (row, column, seed), so that the
generator of the fixtures and the tests build bit-identical inputs without storing them (no dependence on any
library's random stream)."""
import numpy as np


def synth_fp16(rows, cols, seed, scale=1.0):
    """fp16 [rows][cols], values in [-scale, scale), from a 32-bit mix of the indices."""
    i = np.arange(rows, dtype=np.uint64)[:, None]
    j = np.arange(cols, dtype=np.uint64)[None, :]
    h = (i * np.uint64(2654435761) + j * np.uint64(40503) + np.uint64(seed) * np.uint64(2246822519)) & np.uint64(0xFFFFFFFF)
    h ^= h >> np.uint64(15)
    h = (h * np.uint64(2246822519)) & np.uint64(0xFFFFFFFF)
    h ^= h >> np.uint64(13)
    h = (h * np.uint64(3266489917)) & np.uint64(0xFFFFFFFF)
    h ^= h >> np.uint64(16)
    u = (h & np.uint64(0xFFFF)).astype(np.float32) / np.float32(32768.0) - np.float32(1.0)
    return (u * np.float32(scale)).astype(np.float16)
