"""The allocation-free decode attention entry point against the ordinary one.

Some hosts of this library cannot allocate once they are running: they gave all
of the GPU's memory to their own arena at start-up (a later cudaMalloc would
fail, or stall every stream while the driver synchronises the device), or they
may only use memory that was handed to them.  For them
tm_cuda_attention_decode_dev_static keeps its scratch in an array inside the
library instead of taking a caller buffer.  This test drives both entry points
through the C ABI with the same inputs, twice in a row (the second call finds
the array as the first one left it), and expects identical results; it also
checks that a geometry beyond the built-in array is refused, not truncated.
Collected last on purpose, so a failure here cannot hide another test.
"""
import numpy as np
import pytest

from conftest import rel_err
from tuckmill_b200 import cuda, testing as T

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("exact", [True, False])
def test_static_scratch_matches_caller_scratch_twice_in_a_row(ctx, oracle, exact):
    heads, kvh, hd, cap, window, eps = 16, 8, 128, 200, 0, 1e-6
    scale = 1.0 / np.sqrt(np.float32(hd))
    qn = ctx.floats((1 + 0.1 * T.activations(0, 20, hd)).astype(np.float32))
    kn = ctx.floats((1 + 0.1 * T.activations(0, 21, hd)).astype(np.float32))
    inv = ctx.floats(oracle.rope_inv_freq(hd, 1e6))
    plane = kvh * cap * hd * 2
    filled = 150  # positions already in the cache: several key blocks, so partials and counters are used
    kfill = T.activations(1, 1, kvh * cap * hd).astype(np.float16)
    vfill = T.activations(1, 2, kvh * cap * hd).astype(np.float16)
    status = ctx.buffer(4, shared=True)
    status.zero()
    scratch = ctx.buffer(cuda.decode_attention_scratch_bytes(heads, kvh, hd, cap))
    scratch.zero()
    launches0 = ctx.kernel_launches()
    for call in range(2):
        pos = filled + call
        q = T.activations(10 + call, 30, heads * hd)
        k = T.activations(10 + call, 31, kvh * hd)
        v = T.activations(10 + call, 32, kvh * hd)
        outs, caches = [], []
        for use_static in (False, True):
            kc, vc = ctx.from_array(kfill), ctx.from_array(vfill)
            pos_buf = ctx.from_array(np.array([pos], np.uint32))
            out = ctx.buffer(heads * hd * 4)
            args = (ctx.floats(q), ctx.floats(k), ctx.floats(v), qn, kn, inv, kc, vc, out)
            tail = (pos_buf, 0, status, heads, kvh, hd, hd, cap, window, eps, scale, exact)
            if use_static:
                ctx.attention_decode_dev_static(*args, *tail)
            else:
                ctx.attention_decode_dev(*args, scratch, *tail)
            ctx.fence()
            outs.append(out.download(0, heads * hd * 4, np.float32))
            caches.append((kc.download(0, plane), vc.download(0, plane)))
        # same kernels, same inputs: the tolerance of the other GPU tests is the reference's
        # 1e-4 rule, and here the two entry points agree to the bit
        assert rel_err(outs[1], outs[0]) <= 1e-4
        np.testing.assert_array_equal(outs[1], outs[0])
        np.testing.assert_array_equal(caches[1][0], caches[0][0])
        np.testing.assert_array_equal(caches[1][1], caches[0][1])
        assert np.all(np.isfinite(outs[1])) and float(np.max(np.abs(outs[1]))) > 0
    assert int(status.download(0, 4, np.uint32)[0]) == 0
    assert ctx.kernel_launches() >= launches0 + 4


@pytest.mark.parametrize("exact", [True, False])
def test_static_scratch_after_a_call_of_another_geometry(ctx, oracle, exact):
    """Callers that cannot allocate also cannot give each model its own scratch: every geometry shares
    the one built-in array.  A call's arrival counters then land where an earlier call of another
    geometry left partial results, so each call has to clear the words it is about to count in.  Here a
    wide geometry runs first and a narrower one, whose counters fall inside the first one's partials,
    second; the second must still agree with the caller-scratch entry point to the bit."""
    eps = 1e-6
    geometries = [(16, 8, 128, 200, 199), (4, 2, 128, 96, 70), (8, 8, 128, 200, 130)]
    status = ctx.buffer(4, shared=True)
    status.zero()
    for n, (heads, kvh, hd, cap, pos) in enumerate(geometries):
        scale = 1.0 / np.sqrt(np.float32(hd))
        qn = ctx.floats((1 + 0.1 * T.activations(0, 20, hd)).astype(np.float32))
        kn = ctx.floats((1 + 0.1 * T.activations(0, 21, hd)).astype(np.float32))
        inv = ctx.floats(oracle.rope_inv_freq(hd, 1e6))
        kfill = T.activations(2 + n, 1, kvh * cap * hd).astype(np.float16)
        vfill = T.activations(2 + n, 2, kvh * cap * hd).astype(np.float16)
        q, k, v = (T.activations(20 + n, t, w * hd) for t, w in ((30, heads), (31, kvh), (32, kvh)))
        outs = []
        for use_static in (False, True):
            kc, vc = ctx.from_array(kfill), ctx.from_array(vfill)
            pos_buf = ctx.from_array(np.array([pos], np.uint32))
            out = ctx.buffer(heads * hd * 4)
            args = (ctx.floats(q), ctx.floats(k), ctx.floats(v), qn, kn, inv, kc, vc, out)
            tail = (pos_buf, 0, status, heads, kvh, hd, hd, cap, 0, eps, scale, exact)
            if use_static:
                ctx.attention_decode_dev_static(*args, *tail)
            else:
                scratch = ctx.buffer(cuda.decode_attention_scratch_bytes(heads, kvh, hd, cap))
                scratch.zero()
                ctx.attention_decode_dev(*args, scratch, *tail)
            ctx.fence()
            outs.append(out.download(0, heads * hd * 4, np.float32))
        assert rel_err(outs[1], outs[0]) <= 1e-4
        np.testing.assert_array_equal(outs[1], outs[0], err_msg=f"geometry {n}: {heads} heads, capacity {cap}")
    assert int(status.download(0, 4, np.uint32)[0]) == 0


def test_static_scratch_refuses_what_does_not_fit(ctx):
    limit = cuda.decode_attention_static_max_scratch()
    heads, kvh, hd = 64, 8, 256
    cap = 1
    while cuda.decode_attention_scratch_bytes(heads, kvh, hd, cap) <= limit:
        cap *= 2
    small = ctx.buffer(256)
    big_q, big_kv = ctx.buffer(heads * hd * 4), ctx.buffer(kvh * hd * 4)
    with pytest.raises(cuda.CudaError) as e:
        ctx.attention_decode_dev_static(big_q, big_kv, big_kv, small, small, small, small, small, big_q, small, 0,
                                        small, heads, kvh, hd, hd, cap, 0, 1e-6, 0.1, True)
    assert e.value.code == -4 and "built-in scratch" in e.value.message
