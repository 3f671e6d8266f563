"""Reader and writer of YTensor's `.yt` container, and the checkpoint loader of the decoder built on it.

The format is the one yt::io::YTensorIO writes (reference src/ytensor_io.inl:458-559 header and index,
:360-400 tensor records, :24-70 strings and arrays, :72-140 zlib):

    "YTENSORF" | version u8 | metadata (u32 length + bytes)
    per tensor: name, type name (strings) | type size i32 | tensor type (string, "dense") |
                shape (u64 byte count + i32 extents) | compress method (string, "" or "zlib") |
                stored size u64 | stored bytes
    index: u64 offset per tensor | tensor count u32          (at the end of the file)

All integers are little endian. Dense tensors are row-major. The reader maps the file and hands out numpy views
(no copy for uncompressed tensors); `to_device` puts one on the GPU as a torch tensor, bfloat16 staying 16-bit.
"""
from __future__ import annotations

import mmap
import struct
import zlib
from pathlib import Path

import numpy as np

MAGIC = b"YTENSORF"
VERSION = 0

# type name in the file -> numpy dtype holding the same bytes (bfloat16 has no numpy dtype: its bits as uint16)
_NUMPY_OF = {"float32": np.float32, "float64": np.float64, "float16": np.float16, "bfloat16": np.uint16,
             "int8": np.int8, "int16": np.int16, "int32": np.int32, "int64": np.int64, "uint8": np.uint8,
             "uint16": np.uint16, "uint32": np.uint32, "uint64": np.uint64, "bool": np.bool_}


class YtFormatError(ValueError):
    pass


class TensorRecord:
    __slots__ = ("name", "type_name", "type_size", "tensor_type", "shape", "compress", "stored_size", "data_offset")

    def __repr__(self):
        return f"TensorRecord({self.name!r}, {self.type_name}, shape={self.shape}, compress={self.compress!r})"


class _Cursor:
    def __init__(self, buf, pos=0):
        self.buf, self.pos = buf, pos

    def take(self, n: int) -> bytes:
        if n < 0 or self.pos + n > len(self.buf):
            raise YtFormatError("truncated .yt file")
        b = self.buf[self.pos:self.pos + n]
        self.pos += n
        return b

    def u8(self):
        return self.take(1)[0]

    def i32(self):
        return struct.unpack("<i", self.take(4))[0]

    def u32(self):
        return struct.unpack("<I", self.take(4))[0]

    def u64(self):
        return struct.unpack("<Q", self.take(8))[0]

    def string(self) -> str:
        return bytes(self.take(self.u32())).decode("utf-8")


class YtFile:
    """Read-only view of a `.yt` file: `names()`, `record(name)`, `load(name)`, `to_device(name, device)`."""

    def __init__(self, path):
        self.path = Path(path)
        self._fh = open(self.path, "rb")
        try:
            self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        except ValueError as e:  # empty file
            self._fh.close()
            raise YtFormatError(f"{self.path}: empty file") from e
        buf = self._map
        cur = _Cursor(buf)
        if bytes(cur.take(8)) != MAGIC:
            raise YtFormatError(f"{self.path}: bad magic")
        self.version = cur.u8()
        if self.version != VERSION:
            raise YtFormatError(f"{self.path}: unsupported version {self.version}")
        self.metadata = cur.string()
        if len(buf) < cur.pos + 4:
            raise YtFormatError("truncated .yt file")
        count = struct.unpack("<I", buf[len(buf) - 4:])[0]
        index_at = len(buf) - 4 - 8 * count
        if index_at < cur.pos:
            raise YtFormatError(f"{self.path}: index of {count} tensors does not fit the file")
        offsets = struct.unpack(f"<{count}Q", buf[index_at:index_at + 8 * count]) if count else ()
        self._records: dict[str, TensorRecord] = {}
        for off in offsets:
            c = _Cursor(buf, off)
            r = TensorRecord()
            r.name, r.type_name, r.type_size, r.tensor_type = c.string(), c.string(), c.i32(), c.string()
            nbytes = c.u64()
            if nbytes % 4:
                raise YtFormatError(f"{r.name}: shape record of {nbytes} bytes")
            r.shape = tuple(struct.unpack(f"<{nbytes // 4}i", c.take(nbytes))) if nbytes else ()
            r.compress, r.stored_size = c.string(), c.u64()
            r.data_offset = c.pos
            if r.data_offset + r.stored_size > index_at:
                raise YtFormatError(f"{r.name}: data runs past the index")
            self._records[r.name] = r

    def names(self) -> list[str]:
        return list(self._records)

    def __contains__(self, name: str) -> bool:
        return name in self._records

    def record(self, name: str) -> TensorRecord:
        try:
            return self._records[name]
        except KeyError:
            raise KeyError(f"{self.path}: no tensor named {name!r}") from None

    def load(self, name: str) -> np.ndarray:
        """The tensor as a numpy array of its shape (bfloat16 as uint16 bit patterns). Uncompressed tensors are
        read-only views of the mapped file."""
        r = self.record(name)
        if r.tensor_type != "dense":
            raise YtFormatError(f"{name}: tensor type {r.tensor_type!r} is not supported (dense only)")
        if r.type_name not in _NUMPY_OF:
            raise YtFormatError(f"{name}: element type {r.type_name!r} is not supported")
        dt = np.dtype(_NUMPY_OF[r.type_name])
        if dt.itemsize != r.type_size:
            raise YtFormatError(f"{name}: type size {r.type_size} does not fit {r.type_name}")
        want = int(np.prod(r.shape, dtype=np.int64)) * dt.itemsize if r.shape else dt.itemsize
        raw = memoryview(self._map)[r.data_offset:r.data_offset + r.stored_size]
        if r.compress == "zlib":
            raw = zlib.decompress(raw, wbits=47)  # zlib or gzip framing, as inflateInit2(15 + 32) accepts
        # any other method name ("zlibfloat" is named in the reference's header, include/ytensor_io.hpp:38-42, but has
        # no implementation there): the reference's checkCompressMethod falls back to "no compression"
        # (src/ytensor_io.inl:11-22), so the bytes are taken as they are
        if len(raw) != want:
            raise YtFormatError(f"{name}: {len(raw)} data bytes for shape {r.shape} of {r.type_name}")
        return np.frombuffer(raw, dtype=dt).reshape(r.shape)

    def to_device(self, name: str, device="cuda"):
        """The tensor on `device` as a torch tensor (bfloat16 tensors as torch.bfloat16)."""
        import torch
        a = self.load(name)
        t = torch.from_numpy(np.array(a, copy=True)).to(device)  # the mapped view is read-only: copy first
        return t.view(torch.bfloat16) if self.record(name).type_name == "bfloat16" else t

    def close(self):
        if getattr(self, "_map", None) is not None:
            try:
                self._map.close()
            except BufferError:  # arrays handed out still point into the mapping
                pass
            self._map = None
        if getattr(self, "_fh", None) is not None:
            self._fh.close()
            self._fh = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


def _string(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<I", len(b)) + b


def write_yt(path, tensors: dict, *, compress: str = "", bfloat16: tuple = (), metadata: str = "") -> None:
    """Writes numpy arrays as a `.yt` file YTensorIO reads. Names in `bfloat16` are uint16 arrays stored as
    bfloat16 tensors. compress: "" or "zlib"; any other name (e.g. "zlibfloat", which the reference names but does not
    implement) is stored uncompressed, as YTensorIO's checkCompressMethod does (src/ytensor_io.inl:11-22)."""
    if compress not in ("", "zlib"):
        compress = ""
    names_of = {np.dtype(v).name: k for k, v in _NUMPY_OF.items() if k != "bfloat16"}
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack("<B", VERSION) + _string(metadata))
        offsets = []
        for name, arr in tensors.items():
            a = np.ascontiguousarray(arr)
            if name in bfloat16:
                if a.dtype != np.uint16:
                    raise ValueError(f"{name}: bfloat16 tensors are given as uint16 bit patterns")
                type_name = "bfloat16"
            else:
                type_name = names_of.get(a.dtype.name)
                if type_name is None:
                    raise ValueError(f"{name}: dtype {a.dtype} has no .yt type")
            data = a.tobytes()
            stored = zlib.compress(data) if compress == "zlib" else data
            offsets.append(f.tell())
            f.write(_string(name) + _string(type_name) + struct.pack("<i", a.dtype.itemsize) + _string("dense"))
            f.write(struct.pack("<Q", 4 * a.ndim) + struct.pack(f"<{a.ndim}i", *a.shape))
            f.write(_string(compress) + struct.pack("<Q", len(stored)) + stored)
        f.write(struct.pack(f"<{len(offsets)}Q", *offsets) + struct.pack("<I", len(offsets)))


def load_qwen3_checkpoint(path, cfg) -> dict:
    """Weights of a converted checkpoint in the layout Qwen3ForCausalLM.load_weights takes.

    Follows qwen3::Qwen3Model::load (reference example/qwen3/src/qwen3.cpp:304-364): the tensor names of the
    checkpoint ("model.layers.N.self_attn.q_proj.weight", ...), q / k / v concatenated into the fused qkv matrix
    and gate / up into gate_up along the output dim, a missing "lm_head.weight" meaning a tied vocabulary matrix.
    Matrices must be stored as bfloat16 (what the device kernels stream); norm weights may be bfloat16 or float32.
    """
    from .qwen3 import bf16_bits_to_f32

    def matrix(f: YtFile, name: str) -> np.ndarray:
        r = f.record(name)
        if r.type_name != "bfloat16" or len(r.shape) != 2:
            raise YtFormatError(f"{name}: expected a 2-D bfloat16 tensor, found {r.type_name} {r.shape}")
        return f.load(name)

    def vector(f: YtFile, name: str) -> np.ndarray:
        a = f.load(name)
        if f.record(name).type_name == "bfloat16":
            return bf16_bits_to_f32(a).astype(np.float32)
        return np.asarray(a, np.float32)

    w: dict = {}
    with YtFile(path) as f:
        w["embed"] = np.array(matrix(f, "model.embed_tokens.weight"))
        w["norm"] = vector(f, "model.norm.weight")
        if "lm_head.weight" in f:
            w["lm_head"] = np.array(matrix(f, "lm_head.weight"))
        for l in range(cfg.num_hidden_layers):
            p = f"model.layers.{l}."
            w[("qkv", l)] = np.concatenate([matrix(f, p + f"self_attn.{n}_proj.weight") for n in "qkv"], axis=0)
            w[("o", l)] = np.array(matrix(f, p + "self_attn.o_proj.weight"))
            w[("gate_up", l)] = np.concatenate([matrix(f, p + "mlp.gate_proj.weight"),
                                                matrix(f, p + "mlp.up_proj.weight")], axis=0)
            w[("down", l)] = np.array(matrix(f, p + "mlp.down_proj.weight"))
            w[("q_norm", l)] = vector(f, p + "self_attn.q_norm.weight")
            w[("k_norm", l)] = vector(f, p + "self_attn.k_norm.weight")
            w[("norm1", l)] = vector(f, p + "input_layernorm.weight")
            w[("norm2", l)] = vector(f, p + "post_attention_layernorm.weight")
    H, D = cfg.hidden_size, cfg.head_dim
    want = {"embed": (cfg.vocab_size, H), ("qkv", 0): ((cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * D, H),
            ("o", 0): (H, cfg.num_attention_heads * D), ("gate_up", 0): (2 * cfg.intermediate_size, H),
            ("down", 0): (H, cfg.intermediate_size)}
    for key, shape in want.items():
        if tuple(w[key].shape) != shape:
            raise YtFormatError(f"{key}: shape {tuple(w[key].shape)} does not fit the configuration ({shape})")
    return w
