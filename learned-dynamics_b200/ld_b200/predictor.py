"""Host-side mirror of the rollout loop around the denoiser: ModelState and ModelPredictor.predict
(managan/predictor.py:129-176) and the trajectory file format (managan/statefiles.py:16-42).

ModelPredictor.predict keeps the reference's contract (it MUTATES `state`, returns a ModelState of
size (L, *state.size)). Two things differ underneath:

* the trajectory buffer lives on the device and frames are copied into it by the stream that ran
  the step, as in the reference; optionally every frame is also streamed to pinned host memory on a
  second stream while the next step runs (`host_frames=True`), so that a rollout that is written
  to disk does not end with one large blocking device-to-host copy;
* a `counter` tensor, when given, receives the number of edge messages the steps processed.

The file format is the reference's: a "!III" header with the three subfile lengths, then
pickle(metadata), pickle(shape) and the positions as an .npy image."""
import pickle
from io import BytesIO
from struct import pack, unpack

import numpy as np
import torch


def _assert_shapes_compatible(base_shape, shape):
    assert len(base_shape) == len(shape), "number of dimensions does not match"
    for d_base, d in zip(base_shape, shape):
        assert d_base == d or d_base == -1, f"dimension mismatch {d_base} != {d}"


class ModelState:
    """positions `x` of size (*size, *shape), e.g. size (batch,) or (time, batch), shape (atoms, 3)"""

    def __init__(self, shape, x, **kwargs):
        shape = tuple(shape)
        ndims = len(shape)
        self._size = x.shape[:-ndims]
        _assert_shapes_compatible(shape, tuple(x.shape[-ndims:]))
        self._shape = x.shape[-ndims:]  # torch.Size, as the reference keeps (and pickles) it
        self._x = x
        self.kwargs = kwargs

    @property
    def size(self):
        return self._size

    @property
    def shape(self):
        return self._shape

    @property
    def x(self):
        return self._x

    @property
    def x_npy(self):
        return self._x.cpu().numpy()

    @property
    def metadata(self):
        return self.kwargs.get("metadata")

    def __getitem__(self, key):
        return ModelState(self.shape, self._x[key], **self.kwargs)

    def expand(self, n, dim):
        assert dim <= len(self.size), f"can't unsqueeze dim {dim} for State of shape {self.size}"
        full = tuple(self.size) + tuple(self.shape)
        full = full[:dim] + (n,) + full[dim:]
        return ModelState(self.shape, self._x.unsqueeze(dim).expand(*full).clone(), **self.kwargs)

    def reshape(self, *newsize):
        assert int(np.prod(newsize)) == int(np.prod(self.size)), f"can't reshape {self.size} to {newsize}"
        return ModelState(self.shape, self._x.reshape(*(tuple(newsize) + tuple(self.shape))), **self.kwargs)

    def to_model_predictor_state(self):
        return ModelState(self.shape, self._x.clone(), **self.kwargs)


class ModelPredictor:
    """predict(L, state): L applications of model.predict, each one sampled dt step of every system."""

    def __init__(self, model, host_frames=False):
        if hasattr(model, "set_eval"):
            model.set_eval(True)
        self.model = model
        self.host_frames = host_frames
        self.last_host_trajectory = None
        self._copy_stream = None

    def predict(self, L, state, ret=True, counter=None):
        """MUTATES state"""
        x = state._x
        trajectory = torch.zeros(L, *state.size, *state.shape, dtype=x.dtype, device=x.device) if ret else None
        host = None
        if self.host_frames and x.is_cuda:
            host = torch.empty((L,) + tuple(x.shape), dtype=x.dtype, pin_memory=True)
            if self._copy_stream is None:
                self._copy_stream = torch.cuda.Stream(device=x.device)
            main = torch.cuda.current_stream(x.device)
            staged = [torch.empty_like(x), torch.empty_like(x)]
            free = [torch.cuda.Event(), torch.cuda.Event()]
        with torch.no_grad():
            for i in range(L):
                new_x = self.model.predict(state) if counter is None else self.model.predict(state, counter=counter)
                x[:] = new_x
                if ret:
                    trajectory[i] = new_x
                if host is not None:
                    # frame i leaves through a staging copy so that step i+1 may overwrite x at once
                    slot = i & 1
                    if i >= 2:
                        main.wait_event(free[slot])
                    staged[slot].copy_(x)
                    ready = torch.cuda.Event()
                    ready.record(main)
                    with torch.cuda.stream(self._copy_stream):
                        self._copy_stream.wait_event(ready)
                        host[i].copy_(staged[slot], non_blocking=True)
                        free[slot].record(self._copy_stream)
        if host is not None:
            self._copy_stream.synchronize()
            self.last_host_trajectory = host
        if x.is_cuda:
            from . import ops
            ops.check_tc_status(x.device, block=True)   # the trajectory is only handed out if no kernel gave up on a wait
        if ret:
            return ModelState(state.shape, trajectory, **state.kwargs)


def save_state_to_file(file, state):
    """three length-prefixed subfiles: pickled metadata, pickled shape, positions as .npy"""
    x_bytes = BytesIO()
    np.save(x_bytes, state.x_npy, allow_pickle=False)
    subfiles = [pickle.dumps(state.metadata), pickle.dumps(state.shape), x_bytes.getvalue()]
    file.write(pack("!III", *[len(sub) for sub in subfiles]))
    for sub in subfiles:
        file.write(sub)


def save_trajectory_to_file(file, shape, frames, metadata=None):
    """the same file image from a host array (e.g. ModelPredictor.last_host_trajectory) without a
    second copy through a device tensor"""
    arr = frames.numpy() if isinstance(frames, torch.Tensor) else np.asarray(frames)
    _assert_shapes_compatible(tuple(shape), tuple(arr.shape[-len(shape):]))
    x_bytes = BytesIO()
    np.save(x_bytes, arr, allow_pickle=False)
    subfiles = [pickle.dumps(metadata), pickle.dumps(torch.Size(arr.shape[-len(shape):])), x_bytes.getvalue()]
    file.write(pack("!III", *[len(sub) for sub in subfiles]))
    for sub in subfiles:
        file.write(sub)


def read_state_from_file(file, device="cuda"):
    lengths = unpack("!III", file.read(12))
    subfiles = [file.read(n) for n in lengths]
    metadata = pickle.loads(subfiles[0])
    shape = pickle.loads(subfiles[1])
    x_npy = np.load(BytesIO(subfiles[2]), allow_pickle=False)
    return ModelState(shape, torch.tensor(x_npy, device=device), metadata=metadata)
