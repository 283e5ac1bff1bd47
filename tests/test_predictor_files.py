"""Trajectory file image (managan/statefiles.py:16-42) and the ModelState container: the writer must
produce the reference's bytes exactly and the reader must return what was written. Host logic only."""
import io

import numpy as np
import torch

from ld_b200 import predictor as P


def test_writer_reproduces_reference_bytes(golden):
    s = golden["statefile"]
    buf = io.BytesIO()
    P.save_state_to_file(buf, P.ModelState(s["shape"], s["x"], metadata=s["metadata"]))
    assert np.array_equal(np.frombuffer(buf.getvalue(), dtype=np.uint8), s["image"])
    buf2 = io.BytesIO()
    P.save_trajectory_to_file(buf2, s["shape"], s["x"], metadata=s["metadata"])
    assert buf2.getvalue() == buf.getvalue()


def test_reader_round_trip_and_state_algebra(golden):
    s = golden["statefile"]
    state = P.read_state_from_file(io.BytesIO(s["image"].tobytes()), device="cpu")
    assert state.size == (3, 2) and state.shape == (5, 3) and state.metadata == s["metadata"]
    assert torch.equal(state.x, s["x"])
    assert torch.equal(state[1].x, s["x"][1]) and state[1].size == (2,)
    e = state[0].expand(4, 1)
    assert e.size == (2, 4) and torch.equal(e.x[:, 2], s["x"][0])
    assert state.reshape(6).size == (6,)
    c = state.to_model_predictor_state()
    c.x[:] = 0
    assert state.x.abs().max() > 0


def test_empty_trajectory_round_trip():
    buf = io.BytesIO()
    P.save_state_to_file(buf, P.ModelState((4, 3), torch.zeros(0, 2, 4, 3)))
    back = P.read_state_from_file(io.BytesIO(buf.getvalue()), device="cpu")
    assert back.size == (0, 2) and back.shape == (4, 3) and back.metadata is None
