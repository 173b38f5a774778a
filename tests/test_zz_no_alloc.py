"""The allocation-free C entry point of the SDE step agrees with the tensor entry point.

Collected last (file name) so that it also runs after every other GPU test has used the
extension; it passes on its own as well.
"""

import ctypes

import pytest
import torch


def _load_symbol():
    import visionrl_b200._C as ext_module

    lib = ctypes.CDLL(ext_module.__file__)
    fn = lib.vrl_sde_step_noalloc
    fp = ctypes.c_void_p
    fn.argtypes = [fp] * 11 + [ctypes.c_int, ctypes.c_int64, ctypes.c_int, ctypes.c_int, fp,
                               ctypes.c_char_p, ctypes.c_size_t]
    fn.restype = ctypes.c_int
    return fn


def _call(fn, v, x, a, b, scale, dt, prev, noise, deterministic, gaussian):
    batch = v.shape[0]
    n = v.numel() // batch
    nxt, mean = torch.empty_like(v), torch.empty_like(v)
    logp = torch.empty(batch, device=v.device)
    err = ctypes.create_string_buffer(256)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)  # noqa: E731
    rc = fn(ptr(v), ptr(x), ptr(a), ptr(b), ptr(scale), ptr(dt), ptr(prev), ptr(noise), ptr(nxt),
            ptr(mean), ptr(logp), batch, n, int(deterministic), int(gaussian),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), err, len(err))
    return rc, err.value.decode(), nxt, logp, mean


@pytest.mark.gpu
def test_noalloc_entry_matches_tensor_entry_twice():
    from visionrl_b200.ops import _ext

    ext = _ext.load()
    fn = _load_symbol()
    torch.manual_seed(0)
    for shape in [(6, 16, 64, 64), (3, 4, 9, 30, 52)]:
        v = torch.randn(*shape, device="cuda")
        x = torch.randn_like(v)
        noise = torch.randn_like(v)
        a, b, scale, dt = (torch.rand(shape[0], device="cuda") + 0.2 for _ in range(4))
        ref_next, ref_logp, ref_mean = ext.sde_step_fwd(v, x, a, b, scale, dt, None, noise, False, True)
        for _ in range(2):          # two calls in a row share the scratch array
            rc, msg, nxt, logp, mean = _call(fn, v, x, a, b, scale, dt, None, noise, False, True)
            torch.cuda.synchronize()
            assert rc == 0, msg
            assert torch.allclose(nxt, ref_next, atol=1e-6, rtol=1e-6)
            assert torch.allclose(mean, ref_mean, atol=1e-6, rtol=1e-6)
            assert torch.allclose(logp, ref_logp, atol=1e-5, rtol=1e-5)
        # replay form: next sample given
        ref2 = ext.sde_step_fwd(v, x, a, b, scale, dt, ref_next, None, False, True)
        rc, msg, nxt, logp, mean = _call(fn, v, x, a, b, scale, dt, ref_next, None, False, True)
        torch.cuda.synchronize()
        assert rc == 0, msg
        assert torch.allclose(logp, ref2[1], atol=1e-5, rtol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("deterministic,gaussian", [(False, True), (True, True), (False, False)])
def test_noalloc_entry_tail_unaligned_and_modes(deterministic, gaussian):
    """Sizes that are no multiple of four, pointers offset by 4 bytes (the scalar path), the
    deterministic step and the cps score all agree with the tensor entry point, twice."""
    from visionrl_b200.ops import _ext

    ext = _ext.load()
    fn = _load_symbol()
    torch.manual_seed(1)
    batch, n = 5, 4099 * 3 + 1            # n % 4 != 0, several blocks per sample
    def offset(t):                        # same values, storage shifted by one float (4 bytes)
        buf = torch.empty(t.numel() + 1, device="cuda")
        buf[1:].copy_(t.reshape(-1))
        return buf[1:].view(t.shape)
    v = offset(torch.randn(batch, n, device="cuda"))
    x = offset(torch.randn(batch, n, device="cuda"))
    noise = offset(torch.randn(batch, n, device="cuda"))
    assert v.data_ptr() % 16 != 0
    a, b, scale, dt = (torch.rand(batch, device="cuda") + 0.2 for _ in range(4))
    ref_next, ref_logp, ref_mean = ext.sde_step_fwd(v.contiguous(), x.contiguous(), a, b, scale, dt,
                                                    None, noise.contiguous(), deterministic, gaussian)
    for _ in range(2):
        rc, msg, nxt, logp, mean = _call(fn, v, x, a, b, scale, dt, None, noise, deterministic, gaussian)
        torch.cuda.synchronize()
        assert rc == 0, msg
        assert torch.allclose(nxt, ref_next, atol=1e-6, rtol=1e-6)
        assert torch.allclose(mean, ref_mean, atol=1e-6, rtol=1e-6)
        assert torch.allclose(logp, ref_logp, atol=1e-5, rtol=1e-5)


@pytest.mark.gpu
def test_noalloc_entry_rejects_absurd_length():
    """A length whose block count does not fit 32 bits is refused as too large (rc 2), not wrapped."""
    fn = _load_symbol()
    dummy = torch.zeros(8, device="cuda")
    err = ctypes.create_string_buffer(256)
    p = ctypes.c_void_p(dummy.data_ptr())
    rc = fn(p, p, p, p, p, p, None, p, p, p, p, 1, (1 << 44) + 5, 0, 1, None, err, len(err))
    assert rc == 2, err.value


@pytest.mark.gpu
def test_noalloc_entry_rejects_oversized_problem():
    fn = _load_symbol()
    batch, n = 20, 4096 * 4000          # 20 * 4000 partial sums > 65536
    dummy = torch.zeros(8, device="cuda")
    err = ctypes.create_string_buffer(256)
    p = ctypes.c_void_p(dummy.data_ptr())
    rc = fn(p, p, p, p, p, p, None, p, p, p, p, batch, n, 0, 1, None, err, len(err))
    assert rc == 2
    assert b"scratch" in err.value
