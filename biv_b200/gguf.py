"""A minimal reader of the GGUF container, enough to hand a qwen35moe layer's MoE
tensors to ``Moe`` / ``EpMoe`` straight from a model file (memory-mapped, no copy).

Mirrors what the reference's loader does for this path: the container
(engine/src/gguf.rs:21-22 magic and version, 200-212 and 263-321 key/values,
tensor infos and the aligned data section), the tensor names of a block
(engine/src/gguf/tensors.rs:112-131) and ``Loader::ffn`` (engine/src/model.rs:
377-421), including the fused ``ffn_gate_up_exps`` tensor (gate rows then up rows
per expert, model.rs:389-399).  Nothing else of the file is interpreted.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from typing import Dict, List, Tuple

import numpy as np

from .workloads import ExpertStack, MoeLayer, row_size, F32

MAGIC = 0x46554747          # "GGUF", little-endian
(T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64) = range(13)
_SCALAR = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f",
           T_BOOL: "<?", T_U64: "<Q", T_I64: "<q", T_F64: "<d"}


class GgufError(ValueError):
    pass


@dataclass
class TensorInfo:
    name: str
    ty: int                  # ggml type id
    dims: Tuple[int, ...]    # fastest dimension first: [cols, rows, experts]
    offset: int              # bytes from the start of the data section


class _Cursor:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt):
        v = struct.unpack_from(fmt, self.buf, self.pos)[0]
        self.pos += struct.calcsize(fmt)
        return v

    def string(self):
        n = self.take("<Q")
        if self.pos + n > len(self.buf):
            raise GgufError("string runs past the end of the file")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, ty):
        if ty in _SCALAR:
            return self.take(_SCALAR[ty])
        if ty == T_STR:
            return self.string()
        if ty == T_ARR:
            et, n = self.take("<I"), self.take("<Q")
            if et in _SCALAR and et != T_BOOL:      # bulk-read numeric arrays (token tables are long)
                fmt = _SCALAR[et][1]
                size = struct.calcsize(fmt)
                a = np.frombuffer(self.buf, dtype=np.dtype("<" + fmt), count=n, offset=self.pos)
                self.pos += n * size
                return a
            return [self.value(et) for _ in range(n)]
        raise GgufError(f"unknown metadata value type {ty}")


class GgufFile:
    """The key/values and tensor table of one GGUF file; tensor bytes are views of
    the memory map."""

    def __init__(self, path: str):
        self._f = open(path, "rb")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        c = _Cursor(self._map)
        if len(self._map) < 24 or c.take("<I") != MAGIC:
            raise GgufError("not a GGUF file")
        self.version = c.take("<I")
        if self.version not in (2, 3):
            raise GgufError(f"GGUF version {self.version} is not supported")
        n_tensors, n_kv = c.take("<Q"), c.take("<Q")
        self.metadata: Dict[str, object] = {}
        for _ in range(n_kv):
            key = c.string()
            self.metadata[key] = c.value(c.take("<I"))
        self.tensors: Dict[str, TensorInfo] = {}
        for _ in range(n_tensors):
            name = c.string()
            nd = c.take("<I")
            dims = tuple(c.take("<Q") for _ in range(nd))
            ty, off = c.take("<I"), c.take("<Q")
            self.tensors[name] = TensorInfo(name, ty, dims, off)
        align = int(self.metadata.get("general.alignment", 32))
        self.data_start = -(-c.pos // align) * align
        self._bytes = np.frombuffer(self._map, dtype=np.uint8)

    def close(self):
        self._bytes = None
        try:
            self._map.close()
        except BufferError:      # views of the map are still alive; the OS unmaps at exit
            pass
        self._f.close()

    def nbytes(self, t: TensorInfo) -> int:
        rows = 1
        for d in t.dims[1:]:
            rows *= d
        return rows * row_size(t.ty, t.dims[0])

    def data(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        lo = self.data_start + t.offset
        hi = lo + self.nbytes(t)
        if hi > self._bytes.size:
            raise GgufError(f"tensor {name} runs past the end of the file")
        return self._bytes[lo:hi]

    # ---- the MoE feed-forward of block i, as Loader::ffn gathers it -----------------
    def _need(self, name: str, dims: List[int]) -> TensorInfo:
        if name not in self.tensors:
            raise GgufError(f"missing tensor {name}")
        t = self.tensors[name]
        if list(t.dims) != dims:
            raise GgufError(f"tensor {name} has dims {list(t.dims)}, expected {dims}")
        return t

    def moe_config(self) -> dict:
        arch = self.metadata.get("general.architecture")
        if arch != "qwen35moe":
            raise GgufError(f"architecture {arch!r} has no mixture-of-experts feed-forward here")
        m = self.metadata
        cfg = dict(n_embd=int(m[f"{arch}.embedding_length"]), n_expert=int(m[f"{arch}.expert_count"]),
                   k=int(m[f"{arch}.expert_used_count"]), ff=int(m[f"{arch}.expert_feed_forward_length"]),
                   ff_sh=int(m.get(f"{arch}.expert_shared_feed_forward_length", 0)))
        if not 1 <= cfg["k"] <= cfg["n_expert"]:       # model.rs:108-112
            raise GgufError("expert_used_count not in 1..=expert_count")
        return cfg

    def moe_layer(self, i: int) -> MoeLayer:
        c = self.moe_config()
        e, n, ff, sff = c["n_embd"], c["n_expert"], c["ff"], c["ff_sh"]
        p = f"blk.{i}."

        def stack(name, cols, rows, count, offset=0, stride_rows=None):
            t = self._need(name, [cols, stride_rows or rows, count] if count > 1 or name.endswith("_exps.weight")
                           else [cols, rows])
            rb = row_size(t.ty, cols)
            return ExpertStack(t.ty, cols, rows, count, self.data(name), (stride_rows or rows) * rb, offset)

        router_t = self._need(p + "ffn_gate_inp.weight", [e, n])
        if router_t.ty != F32:
            raise GgufError("the router is expected in F32")
        router = self.data(p + "ffn_gate_inp.weight").view(np.float32).reshape(n, e)
        if p + "ffn_gate_up_exps.weight" in self.tensors:      # gate rows then up rows, per expert
            name = p + "ffn_gate_up_exps.weight"
            t = self.tensors[name]
            gate = stack(name, e, ff, n, 0, 2 * ff)
            up = stack(name, e, ff, n, ff * row_size(t.ty, e), 2 * ff)
        else:
            gate = stack(p + "ffn_gate_exps.weight", e, ff, n)
            up = stack(p + "ffn_up_exps.weight", e, ff, n)
        down = stack(p + "ffn_down_exps.weight", ff, e, n)
        layer = MoeLayer(e, n, c["k"], ff, sff, router, gate, up, down)
        if sff:
            layer.sh_gate = stack(p + "ffn_gate_shexp.weight", e, sff, 1)
            layer.sh_up = stack(p + "ffn_up_shexp.weight", e, sff, 1)
            layer.sh_down = stack(p + "ffn_down_shexp.weight", sff, e, 1)
            gi = self._need(p + "ffn_gate_inp_shexp.weight", [e])
            if gi.ty != F32:
                raise GgufError("the shared expert's gate vector is expected in F32")
            layer.sh_gate_inp = self.data(p + "ffn_gate_inp_shexp.weight").view(np.float32)
        return layer
