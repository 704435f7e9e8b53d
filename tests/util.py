"""Shared helpers of the GPU parity tests (test infrastructure)."""
import numpy as np
import torch

# Output tolerance stated by the task for this floating-point path: max relative error 1e-2
# (fp32 accumulate, fp16 out).  Two forms are asserted: the error relative to the output's
# scale, and the reference tests' own element-wise criterion |a-b| <= 1e-2 + 1e-2*|b|
# (tests/python/relax/test_codegen_cutlass.py:1609).  In practice the kernels agree with the
# oracle to a few fp16 ulps; a tighter bound is asserted too so that regressions show.
RTOL = 1e-2
ATOL = 1e-2


def assert_close(got, exp, tight=True):
    got = np.asarray(got, dtype=np.float32)
    exp = np.asarray(exp, dtype=np.float32)
    assert got.shape == exp.shape
    assert np.all(np.isfinite(got) == np.isfinite(exp))
    m = np.isfinite(exp)
    scale = max(float(np.max(np.abs(exp[m]))), 1e-6) if m.any() else 1.0
    err = np.abs(got[m] - exp[m])
    assert float(err.max(initial=0.0)) / scale <= RTOL, "max err %g relative to scale %g" % (err.max(), scale)
    assert np.all(err <= ATOL + RTOL * np.abs(exp[m]))
    if tight:
        # fp32 accumulation in a different order + one fp16 rounding: ~2 fp16 ulps of the scale
        assert float(err.max(initial=0.0)) <= 2.5e-3 * scale + 1e-6, (err.max(), scale)


def bits16(t):
    if isinstance(t, torch.Tensor):
        t = t.detach().cpu().numpy()
    return np.ascontiguousarray(t, dtype=np.float16).view(np.uint16)


def to_dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.view(dtype) if t.element_size() == torch.empty(0, dtype=dtype).element_size() else t.to(dtype)
    return t.cuda()


def u32_to_dev(w):
    """uint32 numpy -> int32 CUDA tensor with the same bits (torch's uint32 support is partial)."""
    return torch.from_numpy(np.ascontiguousarray(w).view(np.int32)).cuda()
