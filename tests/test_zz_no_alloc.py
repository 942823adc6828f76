"""The allocation-free column-sum entry point against the executable path, through the C ABI.

Collected last on purpose: a run that stops at the first failure has then already run every other
test.  The entry point serves callers that are not allowed to allocate device memory (they were
handed fixed buffers, or sit in a region where the allocator is off limits); its scratch is a
static array inside the library, shared by all calls, so the check runs two calls in a row with
different inputs and shapes and requires each to equal the ordinary SUM_TO_SHAPE step bit for bit.
"""
import numpy as np
import pytest

from synaptik_b200 import native
from synaptik_b200.program import F32, GraphBuilder

pytestmark = pytest.mark.gpu


def _executable_column_sums(ctx, data):
    g = GraphBuilder()
    v = g.feed(F32, data.shape)
    g.publish(g.sum_to_shape(v, (data.shape[1],)))
    exe = native.Executable(ctx, g.build())
    src, dst = ctx.upload(data), ctx.buffer(data.shape[1] * 4)
    try:
        exe.run([src], [dst])
        return dst.download(np.float32, (data.shape[1],))
    finally:
        exe.close(); src.close(); dst.close()


def test_static_scratch_column_sums_match_the_executable_path():
    ctx = native.Context(0)
    rng = np.random.default_rng(21)
    try:
        # two calls in a row: the second is smaller and has other values, so anything the first left
        # in the shared scratch would show
        for rows, cols in ((4097, 1000), (513, 130), (1, 7)):
            data = (rng.standard_normal((rows, cols)) * 3).astype(np.float32)
            src, dst = ctx.upload(data), ctx.buffer(cols * 4)
            native.column_sums_no_alloc(ctx, src, rows, cols, dst)
            got = dst.download(np.float32, (cols,))
            want = _executable_column_sums(ctx, data)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
            assert np.allclose(got, data.astype(np.float64).sum(0), rtol=1e-6, atol=1e-4)
            src.close(); dst.close()
        # sizes beyond the static array are refused, and so are wrong extents
        wide = ctx.buffer(4 * 300000)
        out = ctx.buffer(4 * 300000)
        with pytest.raises(native.NativeFailure) as failure:
            native.column_sums_no_alloc(ctx, wide, 1, 300000, out)
        assert failure.value.status == 8
        with pytest.raises(native.NativeFailure) as failure:
            native.column_sums_no_alloc(ctx, wide, 10, 100000, out)
        assert failure.value.status == 5
        wide.close(); out.close()
    finally:
        ctx.close()
