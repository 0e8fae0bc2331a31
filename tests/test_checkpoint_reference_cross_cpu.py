"""`.sneppx` container against the reference's own writer and reader.

``tests/data/golden_reference_writer.sneppx`` was written by the reference's ``CheckpointWriter``
(interface_bindings/checkpoint.py:96-160) with the content of ``_content()``. It is checked always: this repository's
reader must return that content and its writer must reproduce the file byte for byte. When the reference package is
installed under ``baseline/_ref`` its module is loaded from that file and the two implementations are also run against
each other in both directions; otherwise that part is skipped.
"""
import importlib.util
import os

import numpy as np
import pytest

from sneppx_alg_b200.checkpoint.sneppx_format import CheckpointReader, CheckpointWriter, validate_checkpoint

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "data", "golden_reference_writer.sneppx")
REF = os.path.join(os.path.dirname(HERE), "baseline", "_ref", "SneppX_ALG", "interface_bindings", "checkpoint.py")
META = {"names": ["a", "b", "c"], "step": 17, "note": "written by the reference's CheckpointWriter"}


def _content():
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    b = np.arange(10, dtype=np.int64) * 7 - 3
    c = np.array([1.5, -2.25, 1e-3], dtype=np.float16)
    return [(a.tobytes(), (3, 4), 0, (4, 1)), (b.tobytes(), (10,), 5, (1,)), (c.tobytes(), (3,), 2, ())]


def _write(cls, path, parts, meta):
    w = cls(path)
    for data, shape, dtype, strides in parts:
        w.write_tensor(data, shape, dtype, strides)
    w.write_metadata(meta)
    w.close()


def test_reader_returns_the_golden_files_content():
    assert validate_checkpoint(GOLDEN)
    r = CheckpointReader(GOLDEN)
    for i, (data, shape, dtype, _) in enumerate(_content()):
        info = r.tensor_info(i)
        assert tuple(info[0]) == shape and info[1] == dtype and info[2] == len(data)
        assert r.read_tensor(i) == data
    assert r.read_metadata() == META
    r.close()


def test_writer_reproduces_the_golden_file_byte_for_byte(tmp_path):
    out = str(tmp_path / "ours.sneppx")
    _write(CheckpointWriter, out, _content(), META)
    assert open(out, "rb").read() == open(GOLDEN, "rb").read()


@pytest.mark.skipif(not os.path.exists(REF), reason="reference package not installed under baseline/_ref")
def test_both_directions_against_the_installed_reference(tmp_path):
    spec = importlib.util.spec_from_file_location("reference_checkpoint", REF)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    rng = np.random.default_rng(0)
    parts = [(rng.standard_normal((5, 7)).astype(np.float32).tobytes(), (5, 7), 0, (7, 1)),
             (rng.integers(0, 255, 33, dtype=np.uint8).tobytes(), (33,), 6, (1,)),
             (np.float32(2.5).tobytes(), (1,), 0, ()),
             (rng.standard_normal((2, 3, 4)).astype(np.float64).tobytes(), (2, 3, 4), 1, (12, 4, 1))]
    meta = {"model": "x", "shards": [0, 1], "nested": {"k": 1.5}}
    theirs, ours = str(tmp_path / "theirs.sneppx"), str(tmp_path / "ours.sneppx")
    _write(ref.CheckpointWriter, theirs, parts, meta)
    _write(CheckpointWriter, ours, parts, meta)
    assert open(theirs, "rb").read() == open(ours, "rb").read()
    # their reader on our file, our reader on theirs
    r = ref.CheckpointReader(ours)
    assert [r.read_tensor(i) for i in range(len(parts))] == [p[0] for p in parts] and r.read_metadata() == meta
    assert [tuple(rec.shape) for rec in r.records] == [p[1] for p in parts]
    r.close()
    with CheckpointReader(theirs) as q:
        assert [q.read_tensor(i) for i in range(len(parts))] == [p[0] for p in parts] and q.read_metadata() == meta
    assert ref.validate_checkpoint(ours) and validate_checkpoint(theirs)
