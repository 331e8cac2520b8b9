"""Parameter and optimizer-state checkpoints in the safetensors wire format.

The reference saves and loads parameters through ``LayerMap.serialize /
deserialize`` (``src/utils/layer_map.zig:334-484``) with the safetensors format
(8-byte little-endian header length, a JSON header ``{name: {dtype, shape,
data_offsets}}``, then the raw little-endian tensor bytes in header order).
This module writes and reads that format for tensors that live on the device:
a save is one device-to-host copy of the flat parameter (and Adam state)
buffers, a load the reverse.  Checkpoints are not on the timed path.
"""
from __future__ import annotations

import json
import struct
from typing import Dict

import numpy as np

_DTYPES = {"F32": np.float32, "F64": np.float64, "I32": np.int32, "I64": np.int64, "U32": np.uint32, "U64": np.uint64,
           "U8": np.uint8, "I8": np.int8, "I16": np.int16, "U16": np.uint16, "BOOL": np.bool_, "F16": np.float16}
_NAMES = {np.dtype(v): k for k, v in _DTYPES.items()}


def serialize(tensors: Dict[str, np.ndarray], metadata: Dict[str, str] | None = None) -> bytes:
    header, chunks, off = {}, [], 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, a in tensors.items():
        a = np.ascontiguousarray(a)
        if a.dtype not in _NAMES:
            raise TypeError("unsupported dtype %s for %r" % (a.dtype, name))
        raw = a.astype(a.dtype.newbyteorder("<"), copy=False).tobytes()
        header[name] = {"dtype": _NAMES[a.dtype], "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        chunks.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)  # the data section starts 8-byte aligned
    return struct.pack("<Q", len(hj)) + hj + b"".join(chunks)


def deserialize(data: bytes) -> Dict[str, np.ndarray]:
    if len(data) < 8:
        raise ValueError("not a safetensors buffer")
    (n,) = struct.unpack("<Q", data[:8])
    if 8 + n > len(data):
        raise ValueError("header length %d exceeds the buffer" % n)
    header = json.loads(data[8:8 + n].decode())
    body = memoryview(data)[8 + n:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        dt = np.dtype(_DTYPES[info["dtype"]]).newbyteorder("<")
        a = np.frombuffer(body[b:e], dtype=dt).reshape(info["shape"])
        out[name] = a.astype(dt.newbyteorder("="), copy=True)
    return out


def metadata(data: bytes) -> Dict[str, str]:
    (n,) = struct.unpack("<Q", data[:8])
    return json.loads(data[8:8 + n].decode()).get("__metadata__", {})


# ---------------------------------------------------------------------------
# MLP trainer <-> checkpoint
# ---------------------------------------------------------------------------
def mlp_state(tr) -> Dict[str, np.ndarray]:
    """Named host copies of an MlpTrainer's parameters and, for Adam, its
    moments and step counter (one device-to-host copy per flat buffer)."""
    dev = tr.dev
    out = {}
    flat = dev.to_numpy(tr.params)
    mom = {"adam.m": dev.to_numpy(tr.m), "adam.v": dev.to_numpy(tr.v)} if tr.opt == "adam" else {}
    for l in range(tr.L):
        for kind, seg in (("weight", tr.segments[2 * l]), ("bias", tr.segments[2 * l + 1])):
            shape = (tr.dims[l + 1], tr.dims[l]) if kind == "weight" else (tr.dims[l + 1],)
            off, n = seg
            out["layers.%d.%s" % (l, kind)] = flat[off:off + n].reshape(shape).copy()
            for mname, buf in mom.items():
                out["%s.layers.%d.%s" % (mname, l, kind)] = buf[off:off + n].reshape(shape).copy()
    if tr.opt == "adam":
        out["adam.t"] = np.array([tr.read_t()], np.uint64)
    return out


def save_mlp(tr, path: str) -> None:
    with open(path, "wb") as f:
        f.write(serialize(mlp_state(tr), {"format": "zigrad-b200 mlp", "dims": ",".join(map(str, tr.dims)), "optimizer": tr.opt}))


def load_mlp(tr, path: str) -> None:
    """Restores parameters (and Adam state when both sides have it) into an
    MlpTrainer of the same architecture; the bf16 weight copy is refreshed."""
    with open(path, "rb") as f:
        t = deserialize(f.read())
    dev = tr.dev
    flat = np.empty(tr.n_params, np.float32)
    m, v = np.zeros(tr.n_params, np.float32), np.zeros(tr.n_params, np.float32)
    have_adam = tr.opt == "adam" and "adam.t" in t
    for l in range(tr.L):
        for kind, seg in (("weight", tr.segments[2 * l]), ("bias", tr.segments[2 * l + 1])):
            off, n = seg
            a = t["layers.%d.%s" % (l, kind)]
            if a.size != n:
                raise ValueError("layers.%d.%s has %d elements, the model needs %d" % (l, kind, a.size, n))
            flat[off:off + n] = a.ravel()
            if have_adam:
                m[off:off + n] = t["adam.m.layers.%d.%s" % (l, kind)].ravel()
                v[off:off + n] = t["adam.v.layers.%d.%s" % (l, kind)].ravel()
    dev.mem_transfer_htod(flat, tr.params)
    if have_adam:
        dev.mem_transfer_htod(m, tr.m)
        dev.mem_transfer_htod(v, tr.v)
        tcount = np.array([int(t["adam.t"][0])], np.uint64)
        dev.mem_transfer_htod(tcount, tr.t_dev)
        tr.t = int(tcount[0])
    if tr.bf16:
        dev.cast(tr.params, tr.params_bf16)
    dev.sync()
