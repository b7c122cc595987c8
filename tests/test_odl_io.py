"""`.odl` state-dict files and `.ckpt` checkpoint directories (origindl_b200/odl_io.py) against files written by the
unmodified reference: the committed fixtures of tests/golden/ (made by tests/golden/make_odl_fixtures.py) and, where
the reference library is available, files exchanged with it in both directions.  Follows the reference's own
tests/unit_test/io/test_checkpoint.cpp (SaveAndLoadCheckpoint, SaveAndLoadModelStateDict)."""
from __future__ import annotations

import ctypes
import struct
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).resolve().parent))
from _libs import ref_check, reference  # noqa: E402
from golden import make_odl_fixtures as fx  # noqa: E402

from origindl_b200 import odl_io  # noqa: E402

GOLDEN = Path(__file__).resolve().parent / "golden"


def records(path) -> set:
    """The per-tensor byte records of an .odl file as a set (the reference writes them in hash-map order)."""
    raw = Path(path).read_bytes()
    magic, version, count = struct.unpack_from("<IIQ", raw, 0)
    assert magic == 0x4F444C00 and version == 1
    o, out = 16, set()
    for _ in range(count):
        start = o
        (n,) = struct.unpack_from("<Q", raw, o)
        o += 8 + n
        (rank,) = struct.unpack_from("<Q", raw, o)
        dims = struct.unpack_from(f"<{rank}Q", raw, o + 8)
        o += 8 + 8 * rank
        (code,) = struct.unpack_from("<i", raw, o)
        o += 12
        o += int(np.prod(dims)) * {0: 4, 1: 8, 3: 4}[code]
        out.add(raw[start:o])
    assert o == len(raw)
    return out


def unpack_mlp(packed, sizes) -> dict:
    out, o = {}, 0
    for i in range(len(sizes) - 1):
        for name, shape in ((f"layer_{i}.weight", (sizes[i], sizes[i + 1])), (f"layer_{i}.bias", (1, sizes[i + 1]))):
            n = shape[0] * shape[1]
            out[name] = packed[o:o + n].reshape(shape)
            o += n
    return out


def test_reads_reference_state_file():
    got, devices = odl_io.load(str(GOLDEN / "ref_state.odl"), with_devices=True)
    want = fx.state_tensors()
    assert set(got) == set(want)
    for name, t in want.items():
        assert got[name].dtype == np.float32 and got[name].shape == t.shape
        assert np.array_equal(got[name], t)
        assert devices[name] == (odl_io.DEVICE_CPU, 0)


def test_writer_emits_the_reference_records(tmp_path):
    mine = tmp_path / "mine.odl"
    odl_io.save(fx.state_tensors(), str(mine))
    assert records(mine) == records(GOLDEN / "ref_state.odl")
    assert mine.stat().st_size == (GOLDEN / "ref_state.odl").stat().st_size


def test_dtypes_and_round_trip(tmp_path):
    rng = np.random.default_rng(5)
    sd = {"a": rng.standard_normal((2, 3)).astype(np.float32), "b": rng.standard_normal(4), "c": np.arange(6, dtype=np.int32).reshape(3, 2),
          "empty_name_ok": np.zeros((1, 1), np.float32)}
    p = tmp_path / "t.odl"
    odl_io.save(sd, str(p), device=(odl_io.DEVICE_CUDA, 3))
    got, dev = odl_io.load(str(p), with_devices=True)
    for k in sd:
        assert got[k].dtype == sd[k].dtype and np.array_equal(got[k], sd[k]) and dev[k] == (1, 3)
    with pytest.raises(odl_io.OdlFormatError, match="Unsupported dtype for saving"):
        odl_io.save({"x": np.zeros(3, np.int64)}, str(tmp_path / "bad.odl"))


def test_rejects_what_the_reference_rejects(tmp_path):
    good = (GOLDEN / "ref_state.odl").read_bytes()
    cases = {
        "magic": (b"\x01" + good[1:], "Invalid file format"),
        "version": (good[:4] + struct.pack("<I", 2) + good[8:], "Unsupported file version"),
        "truncated": (good[:-5], "Failed to read tensor data"),
        "count": (good[:12], "Failed to read parameter count"),
    }
    for name, (blob, msg) in cases.items():
        p = tmp_path / f"{name}.odl"
        p.write_bytes(blob)
        with pytest.raises(odl_io.OdlFormatError, match=msg):
            odl_io.load(str(p))
    with pytest.raises(odl_io.OdlFormatError, match="Failed to open file"):
        odl_io.load(str(tmp_path / "missing.odl"))
    # length fields far beyond the file: refused from the file size alone, before anything of that size is allocated
    huge = {
        "huge_name": good[:16] + struct.pack("<Q", 1 << 60) + good[24:],
        "huge_count": good[:8] + struct.pack("<Q", 1 << 62) + good[16:],
    }
    nl = struct.unpack_from("<Q", good, 16)[0]   # first record: name length, name, rank, dims ...
    dim0 = 16 + 8 + nl + 8
    huge["huge_dim"] = good[:dim0] + struct.pack("<Q", 1 << 50) + good[dim0 + 8:]
    for name, blob in huge.items():
        p = tmp_path / f"{name}.odl"
        p.write_bytes(blob)
        with pytest.raises(odl_io.OdlFormatError):
            odl_io.load(str(p))
    # an unsupported dtype code (int64 = 4) in an otherwise valid record
    rec = min(records(GOLDEN / "ref_state.odl"), key=len)
    name_len = struct.unpack_from("<Q", rec, 0)[0]
    rank = struct.unpack_from("<Q", rec, 8 + name_len)[0]
    pos = 8 + name_len + 8 + 8 * rank
    blob = good[:8] + struct.pack("<Q", 1) + rec[:pos] + struct.pack("<i", 4) + rec[pos + 4:]
    p = tmp_path / "dtype.odl"
    p.write_bytes(blob)
    with pytest.raises(odl_io.OdlFormatError, match="Unsupported dtype for loading"):
        odl_io.load(str(p))


def test_reads_reference_checkpoint():
    ck = odl_io.load_checkpoint(str(GOLDEN / "ref_checkpoint.ckpt"))
    m = fx.CKPT_META
    assert (ck.epoch, ck.step, ck.optimizer_type) == (m["epoch"], m["step"], m["optimizer_type"])
    assert ck.loss == pytest.approx(m["loss"])
    for k in ("lr", "beta1", "beta2", "eps"):
        assert ck.optimizer_config[k] == pytest.approx(m[k], rel=1e-6)
    want = unpack_mlp(fx.checkpoint_params(), fx.CKPT_SIZES)
    assert set(ck.model_state_dict) == set(want)
    for k, t in want.items():
        assert np.array_equal(ck.model_state_dict[k], t)
    assert ck.optimizer_state_dict == {}  # the reference never writes optimizer.odl


def test_checkpoint_writer_matches_reference_layout(tmp_path):
    m = fx.CKPT_META
    params = unpack_mlp(fx.checkpoint_params(), fx.CKPT_SIZES)
    opt = {"m_" + k: np.zeros_like(v) for k, v in params.items()}
    opt.update({"step_" + k: np.array([7], np.int32) for k in params})
    ck = odl_io.Checkpoint(params, opt, m["epoch"], m["step"], m["loss"], m["optimizer_type"],
                           {k: m[k] for k in ("lr", "beta1", "beta2", "eps")})
    d = Path(odl_io.save_checkpoint(ck, str(tmp_path / "run.ckpt")))
    assert d == tmp_path / "run" and (d / "model.odl").exists() and (d / "optimizer.odl").exists()
    assert records(d / "model.odl") == records(GOLDEN / "ref_checkpoint" / "model.odl")
    # metadata.json: the same lines (the order of the optimizer_config entries is the reference's hash-map order)
    mine = (d / "metadata.json").read_text().splitlines()
    theirs = (GOLDEN / "ref_checkpoint" / "metadata.json").read_text().splitlines()
    assert mine[:8] == theirs[:8] and mine[-2:] == theirs[-2:]
    assert sorted(s.rstrip(",") for s in mine[8:-2]) == sorted(s.rstrip(",") for s in theirs[8:-2])
    back = odl_io.load_checkpoint(str(tmp_path / "run.ckpt"))
    assert back.epoch == 5 and back.step == 100 and set(back.optimizer_state_dict) == set(opt)
    assert back.optimizer_state_dict["step_layer_0.weight"].dtype == np.int32
    with pytest.raises(odl_io.OdlFormatError, match="Checkpoint directory does not exist"):
        odl_io.load_checkpoint(str(tmp_path / "nothing.ckpt"))


needs_ref = pytest.mark.skipif(reference() is None or not hasattr(reference(), "odlref_save_state"),
                               reason="reference library with the state-dict entry points is not built")


@needs_ref
def test_reference_loads_files_written_here(tmp_path):
    ref = reference()
    sd = fx.state_tensors()
    p = str(tmp_path / "mine.odl").encode()
    odl_io.save(sd, p.decode())
    buf, count = ctypes.create_string_buffer(4096), ctypes.c_int()
    ref_check(ref.odlref_load_state_names(p, buf, 4096, ctypes.byref(count)))
    assert count.value == len(sd) and set(buf.value.decode().split()) == set(sd)
    for name, t in sd.items():
        rank, dims, out = ctypes.c_int(), np.zeros(8, np.int64), np.empty(t.size, np.float32)
        ref_check(ref.odlref_load_state_tensor(p, name.encode(), ctypes.byref(rank), dims, out.ctypes.data_as(ctypes.c_void_p)))
        assert tuple(dims[:rank.value]) == t.shape and np.array_equal(out.reshape(t.shape), t)


@needs_ref
def test_reference_loads_checkpoint_written_here(tmp_path):
    ref = reference()
    params = unpack_mlp(fx.checkpoint_params(), fx.CKPT_SIZES)
    opt = {"m_" + k: np.ones_like(v) for k, v in params.items()}
    ck = odl_io.Checkpoint(params, opt, 3, 42, 1.25, "SGD", {"lr": 0.05})
    path = str(tmp_path / "c.ckpt")
    odl_io.save_checkpoint(ck, path)
    epoch, step, loss, n = ctypes.c_int(), ctypes.c_int(), ctypes.c_float(), ctypes.c_int()
    name, cfg = ctypes.create_string_buffer(64), np.zeros(4, np.float32)
    ref_check(ref.odlref_load_checkpoint_meta(path.encode(), ctypes.byref(epoch), ctypes.byref(step), ctypes.byref(loss),
                                              name, 64, cfg, ctypes.byref(n)))
    assert (epoch.value, step.value, loss.value, name.value, n.value) == (3, 42, 1.25, b"SGD", 4)
    assert cfg[0] == np.float32(0.05) and cfg[1] == -1.0


@needs_ref
def test_fixtures_are_what_the_reference_writes_today(tmp_path):
    fx.ref_save_state(reference(), str(tmp_path / "s.odl"), fx.state_tensors())
    assert records(tmp_path / "s.odl") == records(GOLDEN / "ref_state.odl")
