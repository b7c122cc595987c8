"""Reader / writer of the reference's `.odl` state-dict files and `.ckpt` checkpoint directories.

File format (src/io/model_io.cpp:114-273), little endian, `size_t` = 8 bytes:

    u32 magic 0x4F444C00 ("ODL\\0") | u32 version 1 | u64 tensor count
    per tensor: u64 name length, name bytes | u64 rank, u64 dims[rank] | i32 dtype | i32 device type, i32 device index
                | raw values (float32, float64 or int32 only, like the reference)

dtype codes are the reference's DataType enum (include/origin/mat/basic_types.h:19-27): 0 float32, 1 float64, 3 int32;
device type 0 = CPU, 1 = CUDA (basic_types.h:139-143).  The reference writes tensors in the iteration order of an
`unordered_map`, so the order of records carries no meaning; this writer emits them sorted by name.

A checkpoint (src/io/checkpoint.cpp:15-226) is a DIRECTORY -- the given path with a trailing ".ckpt" removed -- holding
`model.odl`, `metadata.json` (written line by line in the reference's exact layout, which its loader parses by
substring search) and, here, `optimizer.odl`: the reference computes that path and never writes the file
(checkpoint.cpp:38-43), so a resumed reference run restarts Adam from zero moments.  This module writes it with the
key scheme of the reference's own optimizer state dict (src/optim/adam.cpp:116-193): `m_<param>`, `v_<param>` float32
tensors and `step_<param>` int32 tensors of shape {1}.  The reference's loader ignores the extra file.
"""
from __future__ import annotations

import os
import struct
from dataclasses import dataclass, field

import numpy as np

MAGIC = 0x4F444C00
VERSION = 1
DTYPE_CODES = {np.dtype(np.float32): 0, np.dtype(np.float64): 1, np.dtype(np.int32): 3}
CODE_DTYPES = {v: k for k, v in DTYPE_CODES.items()}
DEVICE_CPU, DEVICE_CUDA = 0, 1


class OdlFormatError(RuntimeError):
    """The counterpart of the reference's THROW_RUNTIME_ERROR in load() (model_io.cpp:174-270)."""


def save(state_dict: dict[str, np.ndarray], filepath: str, device: tuple[int, int] = (DEVICE_CPU, 0)) -> None:
    """origin::save(const StateDict&, path).  `device` is recorded per tensor as the reference records tensor.device()."""
    with open(filepath, "wb") as out:
        out.write(struct.pack("<IIQ", MAGIC, VERSION, len(state_dict)))
        for name in sorted(state_dict):
            t = np.ascontiguousarray(state_dict[name])
            if t.dtype not in DTYPE_CODES:
                raise OdlFormatError(f"Unsupported dtype for saving: {t.dtype}")
            raw = name.encode()
            out.write(struct.pack("<Q", len(raw)))
            out.write(raw)
            out.write(struct.pack("<Q", t.ndim))
            out.write(struct.pack(f"<{t.ndim}Q", *t.shape))
            out.write(struct.pack("<iii", DTYPE_CODES[t.dtype], device[0], device[1]))
            out.write(memoryview(t.reshape(-1)).cast("B"))  # no intermediate copy of the values


def load(filepath: str, with_devices: bool = False):
    """origin::load(path) -> {name: ndarray}; with_devices also returns {name: (device type, index)}."""
    try:
        f = open(filepath, "rb")
    except OSError as e:
        raise OdlFormatError(f"Failed to open file for reading: {filepath}") from e
    with f:
        size = os.fstat(f.fileno()).st_size

        def take(n: int, what: str) -> bytes:
            # a length field of a truncated or corrupt file must not become an allocation: compare with what is left
            if n > size - f.tell():
                raise OdlFormatError(f"Failed to read {what} from file")
            b = f.read(n)
            if len(b) != n:
                raise OdlFormatError(f"Failed to read {what} from file")
            return b

        head = f.read(8)
        if len(head) != 8 or struct.unpack("<I", head[:4])[0] != MAGIC:
            raise OdlFormatError(f"Invalid file format or corrupted file: {filepath}")
        version = struct.unpack("<I", head[4:])[0]
        if version != VERSION:
            raise OdlFormatError(f"Unsupported file version: {version}")
        (count,) = struct.unpack("<Q", take(8, "parameter count"))
        if count > size:  # every record takes more than one byte
            raise OdlFormatError(f"Invalid file format or corrupted file: {filepath}")
        tensors, devices = {}, {}
        for _ in range(count):
            (n,) = struct.unpack("<Q", take(8, "string length"))
            name = take(n, "string data").decode()
            (rank,) = struct.unpack("<Q", take(8, "shape dimensions"))
            if rank > 64:
                raise OdlFormatError(f"Failed to read shape dimensions from file (rank {rank})")
            shape = struct.unpack(f"<{rank}Q", take(8 * rank, "shape dimension"))
            code, dev_type, dev_index = struct.unpack("<iii", take(12, "dtype"))
            if code not in CODE_DTYPES:
                raise OdlFormatError(f"Unsupported dtype for loading: {code}")
            dt = CODE_DTYPES[code]
            n_elem = 1
            for d in shape:
                n_elem *= d
            if n_elem * np.dtype(dt).itemsize > size - f.tell():
                raise OdlFormatError(f"Failed to read tensor data for parameter '{name}' from file")
            arr = np.empty(shape, dtype=dt)
            if f.readinto(memoryview(arr.reshape(-1)).cast("B")) != arr.nbytes:
                raise OdlFormatError(f"Failed to read tensor data for parameter '{name}' from file")
            tensors[name] = arr
            devices[name] = (dev_type, dev_index)
    return (tensors, devices) if with_devices else tensors


@dataclass
class Checkpoint:
    """origin::Checkpoint (include/origin/io/checkpoint.h:13-25) plus the optimizer tensors the reference leaves out."""

    model_state_dict: dict = field(default_factory=dict)
    optimizer_state_dict: dict = field(default_factory=dict)  # m_<param>, v_<param>, step_<param>
    epoch: int = -1
    step: int = -1
    loss: float = 0.0
    optimizer_type: str = ""
    optimizer_config: dict = field(default_factory=dict)


def _ckpt_dir(filepath: str) -> str:
    return filepath[:-5] if len(filepath) > 5 and filepath.endswith(".ckpt") else filepath


def _cxx_float(v: float) -> str:
    """How `ostream << float` prints (default precision 6, %g), which is what the reference's writer emits."""
    return f"{float(np.float32(v)):.6g}"


def save_checkpoint(ck: Checkpoint, filepath: str, device: tuple[int, int] = (DEVICE_CPU, 0)) -> str:
    """origin::save(const Checkpoint&, path): returns the checkpoint directory."""
    d = _ckpt_dir(filepath)
    os.makedirs(d, exist_ok=True)
    save(ck.model_state_dict, os.path.join(d, "model.odl"), device)
    if ck.optimizer_state_dict:
        save(ck.optimizer_state_dict, os.path.join(d, "optimizer.odl"), device)
    lines = ["{", '  "format_version": "1.0",', '  "format_type": "origindl_checkpoint",', f'  "epoch": {int(ck.epoch)},',
             f'  "step": {int(ck.step)},', f'  "loss": {_cxx_float(ck.loss)},',
             f'  "optimizer_type": "{ck.optimizer_type}",', '  "optimizer_config": {']
    body = ",\n".join(f'    "{k}": {_cxx_float(v)}' for k, v in ck.optimizer_config.items())
    with open(os.path.join(d, "metadata.json"), "w") as m:
        m.write("\n".join(lines) + "\n" + body + "\n  }\n}\n")
    return d


def load_checkpoint(filepath: str) -> Checkpoint:
    """origin::load_checkpoint(path), with the reference's line-oriented metadata parser (checkpoint.cpp:96-216)."""
    d = _ckpt_dir(filepath)
    if not os.path.isdir(d):
        raise OdlFormatError(f"Checkpoint directory does not exist: {d}")
    model_path, meta_path = os.path.join(d, "model.odl"), os.path.join(d, "metadata.json")
    if not os.path.exists(model_path):
        raise OdlFormatError(f"Model file not found in checkpoint: {model_path}")
    if not os.path.exists(meta_path):
        raise OdlFormatError(f"Metadata file not found in checkpoint: {meta_path}")
    ck = Checkpoint(model_state_dict=load(model_path))
    opt_path = os.path.join(d, "optimizer.odl")
    if os.path.exists(opt_path):
        ck.optimizer_state_dict = load(opt_path)

    def number(line: str) -> str:
        return line.split(":", 1)[1].strip(" \t,\n")

    with open(meta_path) as m:
        for line in m:
            if ":" not in line:
                continue
            if '"epoch"' in line:
                ck.epoch = int(float(number(line)))
            if '"step"' in line:
                ck.step = int(float(number(line)))
            if '"loss"' in line:
                ck.loss = float(number(line))
            if '"optimizer_type"' in line:
                v = line.split(":", 1)[1]
                a = v.find('"')
                b = v.find('"', a + 1)
                if a >= 0 and b >= 0:
                    ck.optimizer_type = v[a + 1:b]
            for key in ("lr", "beta1", "beta2", "eps"):
                if f'"{key}"' in line:
                    ck.optimizer_config[key] = float(number(line))
    return ck
