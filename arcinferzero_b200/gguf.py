"""GGUF reader for the path's weight tensors: finds a tensor's GGUF rows in a model file and hands them to the library as
they lie in the file (no host-side repacking), the counterpart of the reference's loader (src/gguf.h:306-359,
zero/engine_load.h:85-130).

Layout (GGUF v2/v3, little endian): magic "GGUF", u32 version, u64 tensor count, u64 key count; key-value pairs
(string key, u32 type, value); tensor infos (string name, u32 n_dims, u64 dims[n_dims] innermost first, u32 ggml type,
u64 offset); padding to `general.alignment` (default 32); tensor data at data_start + offset.

Only what the path needs is interpreted: scalar / string / array metadata values are parsed so that they can be
skipped and queried, tensor payloads are returned as uint8 views of a memory map."""
from __future__ import annotations

import mmap
import struct

import numpy as np

MAGIC = 0x46554747
# ggml type -> (elements per block, bytes per block) for the types the path multiplies, plus the plain float types
BLOCK = {0: (1, 4), 1: (1, 2), 30: (1, 2),
         8: (32, 34), 12: (256, 144),                                  # Q8_0, Q4_K
         2: (32, 18), 13: (256, 176), 14: (256, 210), 23: (256, 136)}  # Q4_0, Q5_K, Q6_K, IQ4_XS (src/gguf.h:48-70)
WEIGHT_TYPES = (8, 12, 2, 13, 14, 23)   # the block types izb_weight_create takes
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_MAX_ENTRIES = 1_000_000


class GGUFError(ValueError):
    pass


class GGUFFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        try:
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        except ValueError as e:  # empty file
            self._f.close()
            raise GGUFError(f"{path}: {e}") from None
        self._pos = 0
        self.kv: dict[str, object] = {}
        self.tensors: dict[str, tuple[int, tuple[int, ...], int, int]] = {}  # name -> (type, dims, offset, nbytes)
        try:
            self._parse()
        except (struct.error, IndexError):
            self.close()
            raise GGUFError(f"{path}: truncated") from None
        except GGUFError:
            self.close()
            raise

    # ---- low-level reads, all bounds-checked against the map
    def _rd(self, fmt: str):
        n = struct.calcsize(fmt)
        if self._pos + n > len(self._mm):
            raise GGUFError(f"{self.path}: truncated")
        v = struct.unpack_from(fmt, self._mm, self._pos)[0]
        self._pos += n
        return v

    def _rd_str(self) -> str:
        n = self._rd("<Q")
        if n > len(self._mm) - self._pos:
            raise GGUFError(f"{self.path}: string of {n} bytes runs past the end")
        s = bytes(self._mm[self._pos:self._pos + n])
        self._pos += n
        return s.decode("utf-8", errors="replace")

    def _rd_value(self, t: int):
        if t in _SCALAR:
            return self._rd(_SCALAR[t])
        if t == 8:
            return self._rd_str()
        if t == 9:
            et, n = self._rd("<I"), self._rd("<Q")
            if et == 9 or n > len(self._mm) - self._pos:
                raise GGUFError(f"{self.path}: bad array")
            if et in _SCALAR:  # bulk read of a numeric array
                fmt = _SCALAR[et]
                size = struct.calcsize(fmt)
                if n * size > len(self._mm) - self._pos:
                    raise GGUFError(f"{self.path}: array runs past the end")
                a = np.frombuffer(self._mm, dtype=np.dtype(fmt[1:]).newbyteorder("<"), count=n, offset=self._pos)
                self._pos += n * size
                return a
            return [self._rd_value(et) for _ in range(n)]
        raise GGUFError(f"{self.path}: unknown metadata type {t}")

    def _parse(self) -> None:
        if self._rd("<I") != MAGIC:
            raise GGUFError(f"{self.path}: not a GGUF file")
        ver = self._rd("<I")
        if ver < 2:
            raise GGUFError(f"{self.path}: unsupported GGUF version {ver}")
        nt, nkv = self._rd("<Q"), self._rd("<Q")
        left = len(self._mm) - self._pos
        if nkv > left // 12 or nt > left // 24 or nkv > _MAX_ENTRIES or nt > _MAX_ENTRIES:
            raise GGUFError(f"{self.path}: {nt} tensors / {nkv} keys cannot be in a file of this size")
        for _ in range(nkv):
            key = self._rd_str()
            self.kv[key] = self._rd_value(self._rd("<I"))
        infos = []
        for _ in range(nt):
            name = self._rd_str()
            nd = self._rd("<I")
            if nd > 8:
                raise GGUFError(f"{self.path}: {name}: {nd} dimensions")
            dims = tuple(self._rd("<Q") for _ in range(nd))
            infos.append((name, dims, self._rd("<I"), self._rd("<Q")))
        align = self.kv.get("general.alignment", 32)
        if not isinstance(align, int) or align <= 0 or align > (1 << 20) or align & (align - 1):
            raise GGUFError(f"{self.path}: bad alignment {align!r}")
        self.data_start = (self._pos + align - 1) // align * align
        if nt and self.data_start > len(self._mm):
            raise GGUFError(f"{self.path}: truncated")
        room = len(self._mm) - self.data_start
        for name, dims, typ, off in infos:
            nbytes = -1
            if typ in BLOCK and dims:
                blk, bb = BLOCK[typ]
                if dims[0] % blk:
                    raise GGUFError(f"{self.path}: {name}: row length {dims[0]} is not a multiple of the block of type {typ}")
                n = 1
                for d in dims:
                    n *= d
                nbytes = n // blk * bb
                if off > room or nbytes > room - off:
                    raise GGUFError(f"{self.path}: tensor out of range {name}")
            self.tensors[name] = (typ, dims, off, nbytes)

    # ---- queries
    def tensor(self, name: str) -> tuple[int, tuple[int, ...], np.ndarray]:
        """(ggml type, dims innermost first, uint8 view of the payload) of a tensor of a type listed in BLOCK."""
        if name not in self.tensors:
            raise KeyError(name)
        typ, dims, off, nbytes = self.tensors[name]
        if nbytes < 0:
            raise GGUFError(f"{self.path}: {name}: ggml type {typ} is not one this reader sizes")
        return typ, dims, np.frombuffer(self._mm, dtype=np.uint8, count=nbytes, offset=self.data_start + off)

    def weight_rows(self, name: str) -> tuple[int, np.ndarray, int, int, int]:
        """A block-quantised matrix (dims [K, N]) or stack of matrices ([K, N, n_mats]) of one of WEIGHT_TYPES as (type, rows
        [n_mats * N, row_bytes], N, K, n_mats): exactly what izb_weight_create takes."""
        typ, dims, data = self.tensor(name)
        if typ not in WEIGHT_TYPES:
            raise GGUFError(f"{self.path}: {name}: type {typ} is not one the library multiplies (Q8_0, Q4_K, Q4_0, Q5_K, Q6_K, IQ4_XS)")
        if len(dims) not in (2, 3) or dims[0] % 256:
            raise GGUFError(f"{self.path}: {name}: dims {dims} (need [K, N] or [K, N, n_mats], K a multiple of 256)")
        K, N = dims[0], dims[1]
        n_mats = dims[2] if len(dims) == 3 else 1
        return typ, data.reshape(n_mats * N, -1), N, K, n_mats

    def close(self) -> None:
        mm, self._mm = getattr(self, "_mm", None), None
        if mm is not None:
            try:
                mm.close()
            except BufferError:  # views handed out are still alive: the map goes when they do
                pass
        if getattr(self, "_f", None):
            self._f.close()
            self._f = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def stacked_rows(g: GGUFFile, names: list[str]) -> tuple[int, list[np.ndarray], int]:
    """The tensors `names` of one type and one K as (type, [rows of each], K): what izb_weight_create_stack takes (the
    reference's load_w_stack, zero/engine_load.h:315-339: Q | K | V and gate | up uploaded as one matrix)."""
    parts, typ0, K0 = [], None, None
    for n in names:
        typ, rows, N, K, n_mats = g.weight_rows(n)
        if n_mats != 1:
            raise GGUFError(f"{g.path}: {n}: a stack of matrices cannot be a part of a stacked weight")
        if typ0 is None:
            typ0, K0 = typ, K
        elif (typ, K) != (typ0, K0):
            raise GGUFError(f"{g.path}: {n}: type {typ}, K = {K} against type {typ0}, K = {K0} of the parts before it")
        parts.append(rows)
    if not parts:
        raise GGUFError(f"{g.path}: no tensor names given")
    return typ0, parts, K0


def load_stacked(path: str, names: list[str], device: int = 0):
    """Q | K | V or gate | up of a GGUF file as ONE device weight (izb_weight_create_stack); needs the CUDA library."""
    import arcinferzero_b200 as izb
    with GGUFFile(path) as g:
        typ, parts, K = stacked_rows(g, names)
        return izb.stacked_weight(typ, [np.array(p) for p in parts], K, device=device)


def load_gateup(path: str, gate: str, up: str, device: int = 0):
    """The gate and up tensors (matrices or expert stacks [K, F, n_mats]) of a GGUF file as one interleaved weight
    (izb_weight_create_gateup): one GEMM with store mode 3 computes up * silu(gate).  Needs the CUDA library."""
    import arcinferzero_b200 as izb
    with GGUFFile(path) as g:
        tg, rg, F, K, nm = g.weight_rows(gate)
        tu, ru, Fu, Ku, nmu = g.weight_rows(up)
        if (tg, F, K, nm) != (tu, Fu, Ku, nmu):
            raise GGUFError(f"{path}: {gate} and {up} differ in type or shape")
        return izb.gateup_weight(tg, np.array(rg), np.array(ru), F, K, n_mats=nm, device=device)


def load_weight(path: str, name: str, device: int = 0, row_range=None, col_range=None):
    """Creates the library's device weight (izb_weight) for a tensor of a GGUF file; needs the CUDA library."""
    import arcinferzero_b200 as izb
    with GGUFFile(path) as g:
        typ, rows, N, K, n_mats = g.weight_rows(name)
        return izb.Weight(typ, np.array(rows), N, K, n_mats=n_mats, device=device, row_range=row_range, col_range=col_range)
