"""`.ve` weight checkpoints (crates/vearo/src/checkpoint.rs:10-88) and optimizer-state files written by the library."""
import struct

import numpy as np
import pytest

from vearo_b200 import modelspec as ms

pytestmark = pytest.mark.gpu


def ve_bytes(arrays):
    """The reference's writer restated: u32 count; per tensor u32 rank, u32 dims, u32 element count, f32 data (little endian)."""
    out = [struct.pack("<I", len(arrays))]
    for a in arrays:
        out.append(struct.pack("<I", a.ndim))
        out += [struct.pack("<I", d) for d in a.shape]
        out.append(struct.pack("<I", a.size))
        out.append(np.ascontiguousarray(a, dtype="<f4").tobytes())
    return b"".join(out)


@pytest.fixture(scope="module")
def vb():
    import vearo_b200 as vb
    vb.init(0)
    return vb


def tiny_gpt(vb, seed=0):
    V, T, d, h, L, ff = 64, 16, 32, 4, 2, 64
    params = ms.gpt_params(V, T, d, L, ff, seed=seed)
    m = vb.SimpleGPT(V, T, d, h, L, ff); m.load(params)
    return m, params, (V, T)


def test_checkpoint_file_is_the_reference_format(vb, tmp_path):
    m, params, _ = tiny_gpt(vb)
    path = tmp_path / "w.ve"
    m.save_checkpoint(path)
    assert path.read_bytes() == ve_bytes(params)
    # a file produced by the reference's writer loads: different weights in, same weights out
    other = [p + 1.0 for p in params]
    path.write_bytes(ve_bytes(other))
    m.load_checkpoint(path)
    for t, want in zip(m.parameters(), other):
        assert np.array_equal(t.numpy(), want)


def test_checkpoint_mismatches_are_errors(vb, tmp_path):
    m, params, _ = tiny_gpt(vb)
    path = tmp_path / "bad.ve"
    path.write_bytes(ve_bytes(params[:-1]))
    with pytest.raises(vb.VearoError, match="tensor count does not match"):
        m.load_checkpoint(path)
    wrong = list(params); wrong[0] = np.zeros((wrong[0].shape[0] + 1, wrong[0].shape[1]), np.float32)
    path.write_bytes(ve_bytes(wrong))
    with pytest.raises(vb.VearoError, match="shape does not match"):
        m.load_checkpoint(path)
    path.write_bytes(ve_bytes(params)[:-7])       # truncated
    with pytest.raises(vb.VearoError):
        m.load_checkpoint(path)


def test_resume_reproduces_the_uninterrupted_run(vb, tmp_path):
    """3 steps, save weights + optimizer state, 3 more steps == load into a fresh model and optimizer, 3 steps (bit for bit)."""
    def fresh():
        m, _, (V, T) = tiny_gpt(vb)
        return m, vb.AdamW(m.parameters(), 1e-3, 0.9, 0.999, 1e-8, 0.1), V, T
    m, opt, V, T = fresh()
    batches = [ms.gpt_batch(V, 2, T, seed=i) for i in range(6)]
    for x, y in batches[:3]:
        m.train_step(opt, x, y, 1.0)
    m.save_checkpoint(tmp_path / "w.ve"); opt.save_state(tmp_path / "o.ve")
    straight = [m.train_step(opt, x, y, 1.0) for x, y in batches[3:]]
    m2, opt2, _, _ = fresh()
    m2.load_checkpoint(tmp_path / "w.ve"); opt2.load_state(tmp_path / "o.ve")
    resumed = [m2.train_step(opt2, x, y, 1.0) for x, y in batches[3:]]
    assert straight == resumed
    for a, b in zip(m.parameters(), m2.parameters()):
        assert np.array_equal(a.numpy(), b.numpy())


def test_optimizer_state_file_carries_the_exact_step_and_the_rng_counter(vb, tmp_path):
    """The state file restores the per-call randomness counter (vearo-core/src/tensor.rs:1240-1285) and a step counter beyond
    2^24 exactly, so that a resumed run draws the dropout masks and applies the bias corrections of the uninterrupted one."""
    import ctypes as C
    m, _, _ = tiny_gpt(vb)
    opt = vb.AdamW(m.parameters(), 1e-3, 0.9, 0.999, 1e-8, 0.1)
    L = vb.lib()
    L.vh_opt_handle.restype = C.c_int
    big = (1 << 24) + 12345                                  # not representable as one f32
    vb.vb_check(L.vb_opt_set_step(L.vh_opt_handle(opt.o), C.c_uint32(big)))
    vb.set_rng_counter((1 << 40) + 77)
    opt.save_state(tmp_path / "o.ve")
    vb.set_rng_counter(5)
    opt2 = vb.AdamW(m.parameters(), 1e-3, 0.9, 0.999, 1e-8, 0.1)
    opt2.load_state(tmp_path / "o.ve")
    assert vb.rng_counter() == (1 << 40) + 77
    st, n, step = C.c_uint32(0), C.c_int64(0), C.c_uint32(0)
    vb.vb_check(L.vb_opt_state(L.vh_opt_handle(opt2.o), C.byref(st), C.byref(n), C.byref(step)))
    assert step.value == big
    vb.set_rng_counter(0)


def test_damaged_files_are_refused_before_anything_is_allocated(vb, tmp_path):
    """A foreign or truncated file must not be trusted for its length fields (a count or rank of billions)."""
    import struct
    m, params, _ = tiny_gpt(vb)
    path = tmp_path / "bad.ve"
    path.write_bytes(struct.pack("<I", len(params)) + struct.pack("<I", 0xfffffff0))      # absurd rank
    with pytest.raises(vb.VearoError, match="damaged|shape does not match"):
        m.load_checkpoint(path)
    opt = vb.AdamW(m.parameters(), 1e-3)
    path.write_bytes(struct.pack("<I", 0xffffffff))                                         # absurd tensor count
    with pytest.raises(vb.VearoError, match="damaged"):
        opt.load_state(path)
    path.write_bytes(struct.pack("<III", 1, 1, 1000) + struct.pack("<I", 1000))             # says 1000 floats, holds none
    with pytest.raises(vb.VearoError):
        opt.load_state(path)
