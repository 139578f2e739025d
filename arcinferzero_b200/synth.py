"""Seeded synthetic tensors in GGUF block formats (Q8_0, Q4_K) and a minimal GGUF v3 writer.

The reference benchmarks real model files; none is available offline, so the benchmark configurations are driven by
random tensors with the stated shapes and value distributions:

* activations  f32 ~ N(0, 1)
* Q8_0 weights per 32-block: fp16 d ~ U(0.001, 0.02), 32 int8 ~ U[-127, 127]            (GGUF block: 34 bytes)
* Q4_K weights per 256-superblock: fp16 d, dmin ~ U(0, 0.01), eight 6-bit scales and mins ~ U[0, 63],
  256 4-bit quants ~ U[0, 15]                                                            (GGUF superblock: 144 bytes)

The Q4_K packer is the inverse of the reference's get_scale_min_k4 / decode_sb (src/quants.h:61-69, :91-114).
"""
from __future__ import annotations

import struct

import numpy as np

GGML_Q8_0 = 8
GGML_Q4_K = 12
GGML_Q4_0, GGML_Q5_K, GGML_Q6_K, GGML_IQ4_XS = 2, 13, 14, 23


_SB_BYTES = {GGML_Q4_0: 8 * 18, GGML_Q5_K: 176, GGML_Q6_K: 210, GGML_IQ4_XS: 136}


def sb_bytes(qtype: int) -> int:
    """Bytes of 256 weights in GGUF form (src/gguf.h:48-70)."""
    if qtype == GGML_Q4_K:
        return 144
    if qtype == GGML_Q8_0:
        return 8 * 34
    if qtype in _SB_BYTES:
        return _SB_BYTES[qtype]
    raise ValueError(f"unsupported ggml type {qtype}")


def row_bytes(qtype: int, K: int) -> int:
    if K % 256:
        raise ValueError("K must be a multiple of 256")
    return K // 256 * sb_bytes(qtype)


def pack_q4k(d: np.ndarray, dmin: np.ndarray, sc: np.ndarray, mn: np.ndarray, q: np.ndarray) -> np.ndarray:
    """d, dmin: [R] float16; sc, mn: [R, 8] uint8 (0..63); q: [R, 256] uint8 (0..15) -> [R, 144] uint8."""
    R = d.shape[0]
    out = np.zeros((R, 144), np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(R, 2)
    out[:, 2:4] = dmin.astype(np.float16).view(np.uint8).reshape(R, 2)
    s = np.zeros((R, 12), np.uint8)
    s[:, 0:4] = sc[:, 0:4] & 63
    s[:, 4:8] = mn[:, 0:4] & 63
    s[:, 8:12] = (sc[:, 4:8] & 15) | ((mn[:, 4:8] & 15) << 4)
    s[:, 0:4] |= (sc[:, 4:8] >> 4) << 6
    s[:, 4:8] |= (mn[:, 4:8] >> 4) << 6
    out[:, 4:16] = s
    qq = q.reshape(R, 4, 2, 32)  # chunk j, half (0: low nibble, 1: high nibble), l
    out[:, 16:144] = ((qq[:, :, 0, :] & 15) | ((qq[:, :, 1, :] & 15) << 4)).reshape(R, 128)
    return out


def pack_q8_0(d: np.ndarray, q: np.ndarray) -> np.ndarray:
    """d: [B] float16, q: [B, 32] int8 -> [B, 34] uint8 (GGUF Q8_0 blocks)."""
    B = d.shape[0]
    out = np.empty((B, 34), np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(B, 2)
    out[:, 2:34] = q.view(np.uint8)
    return out


def make_weight(qtype: int, N: int, K: int, seed: int) -> np.ndarray:
    """Random GGUF rows [N, row_bytes] uint8 with the benchmark's distributions."""
    rng = np.random.default_rng(seed)
    if qtype == GGML_Q4_K:
        R = N * (K // 256)
        d = rng.uniform(0.0, 0.01, R).astype(np.float16)
        dmin = rng.uniform(0.0, 0.01, R).astype(np.float16)
        sc = rng.integers(0, 64, (R, 8), dtype=np.uint8)
        mn = rng.integers(0, 64, (R, 8), dtype=np.uint8)
        nib = rng.integers(0, 256, (R, 128), dtype=np.uint8)  # two uniform nibbles per byte
        out = pack_q4k(d, dmin, sc, mn, np.zeros((R, 256), np.uint8))
        out[:, 16:144] = nib
        return out.reshape(N, -1)
    if qtype == GGML_Q8_0:
        B = N * (K // 32)
        d = rng.uniform(0.001, 0.02, B).astype(np.float16)
        q = rng.integers(-127, 128, (B, 32), dtype=np.int8)
        return pack_q8_0(d, q).reshape(N, -1)
    # The further types: every field uniform over its range (their byte layouts: src/quants.h:91-148, :297-312)
    if qtype == GGML_Q4_0:      # 18-byte blocks: fp16 d | 16 bytes of nibbles
        B = N * (K // 32)
        out = np.empty((B, 18), np.uint8)
        out[:, 0:2] = rng.uniform(0.001, 0.02, B).astype(np.float16).view(np.uint8).reshape(B, 2)
        out[:, 2:] = rng.integers(0, 256, (B, 16), dtype=np.uint8)
        return out.reshape(N, -1)
    R = N * (K // 256)
    if qtype == GGML_Q5_K:      # fp16 d, dmin | 12 B 6-bit scales / mins | 32 B fifth bits | 128 B nibbles
        out = np.empty((R, 176), np.uint8)
        out[:, 0:2] = rng.uniform(0.0, 0.01, R).astype(np.float16).view(np.uint8).reshape(R, 2)
        out[:, 2:4] = rng.uniform(0.0, 0.01, R).astype(np.float16).view(np.uint8).reshape(R, 2)
        out[:, 4:] = rng.integers(0, 256, (R, 172), dtype=np.uint8)
        return out.reshape(N, -1)
    if qtype == GGML_Q6_K:      # 128 B low nibbles | 64 B upper bits | 16 int8 scales | fp16 d
        out = np.empty((R, 210), np.uint8)
        out[:, 0:208] = rng.integers(0, 256, (R, 208), dtype=np.uint8)
        out[:, 208:210] = rng.uniform(0.0, 0.001, R).astype(np.float16).view(np.uint8).reshape(R, 2)
        return out.reshape(N, -1)
    if qtype == GGML_IQ4_XS:    # fp16 d | u16 upper scale bits | 4 B scale nibbles | 128 B codebook indices
        out = np.empty((R, 136), np.uint8)
        out[:, 0:2] = rng.uniform(0.0, 0.001, R).astype(np.float16).view(np.uint8).reshape(R, 2)
        out[:, 2:] = rng.integers(0, 256, (R, 134), dtype=np.uint8)
        return out.reshape(N, -1)
    raise ValueError(f"unsupported ggml type {qtype}")


def make_act(M: int, K: int, seed: int) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((M, K), dtype=np.float32)


def _gguf_value(v) -> bytes:
    """u32 type + value of one metadata entry (int -> u32, float -> f32, str, bool, list of ints / strings)."""
    def s8(x: str) -> bytes:
        b = x.encode()
        return struct.pack("<Q", len(b)) + b
    if isinstance(v, bool):
        return struct.pack("<I?", 7, v)
    if isinstance(v, int):
        return struct.pack("<II", 4, v)
    if isinstance(v, float):
        return struct.pack("<If", 6, v)
    if isinstance(v, str):
        return struct.pack("<I", 8) + s8(v)
    if isinstance(v, (list, tuple)):
        if v and isinstance(v[0], str):
            return struct.pack("<IIQ", 9, 8, len(v)) + b"".join(s8(x) for x in v)
        return struct.pack("<IIQ", 9, 5, len(v)) + b"".join(struct.pack("<i", x) for x in v)
    raise TypeError(type(v))


def write_gguf(path: str, tensors: dict[str, tuple], meta: dict | None = None) -> None:
    """Minimal GGUF v3 file (layout of src/gguf.h:306-359): tensors maps name -> (ggml_type, rows_bytes, N, K) or
    (ggml_type, rows_bytes, N, K, n_mats) for a stack of matrices; dims are stored as [K, N] / [K, N, n_mats]; data is
    aligned to general.alignment (default 32); meta: optional key -> int / float / str / bool / list entries."""
    meta = meta or {}
    align = int(meta.get("general.alignment", 32))
    infos, blobs, off = [], [], 0
    for name, spec in tensors.items():
        qtype, data, N, K = spec[:4]
        dims = (K, N) if len(spec) == 4 else (K, N, spec[4])
        b = np.ascontiguousarray(data).view(np.uint8).reshape(-1).tobytes()
        nb = name.encode()
        infos.append(struct.pack("<Q", len(nb)) + nb + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
                     + struct.pack("<I", qtype) + struct.pack("<Q", off))
        pad = (-len(b)) % align
        blobs.append(b + b"\0" * pad)
        off += len(b) + pad
    kvs = b""
    for k, v in meta.items():
        kb = k.encode()
        kvs += struct.pack("<Q", len(kb)) + kb + _gguf_value(v)
    head = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(meta)) + kvs + b"".join(infos)
    head += b"\0" * ((-len(head)) % align)
    with open(path, "wb") as f:
        f.write(head)
        for b in blobs:
            f.write(b)
