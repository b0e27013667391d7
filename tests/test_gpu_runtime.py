"""Device / buffer / pool / encoder behaviour on a GPU (upstream src/lib.rs:211-308, tests/test_graph.rs)."""
import numpy as np
import pytest

import mlx_native_b200 as mx
from oracle import oracle as orc
from tests.gpu_util import MV_TOL, TYPES, Ctx, norm_err, normal_acts, normal_weights

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def single_launch_matvec():
    """These tests count launches and compare runs bit for bit: they use the one-kernel, fixed-summation-order
    mat-vec.  (The tensor-core mat-vec is two launches and adds split tiles up with atomics.)"""
    mx.set_option("qmv", "stream")
    yield
    mx.set_option("qmv", "auto")


@pytest.fixture(scope="module")
def ctx():
    return Ctx()


def test_device_and_buffers(ctx):
    d = ctx.device
    assert "B200" in d.name() or d.sm_count() > 0
    b = d.alloc_buffer(4096, mx.DType.F32, [32, 32])
    assert b.dtype() == mx.DType.F32 and b.shape() == [32, 32] and b.byte_len() == 4096 and b.element_count() == 1024
    assert np.all(b.as_slice(np.float32) == 0)          # new buffers are zero-filled
    b.as_mut_slice(np.float32)[:] = np.arange(1024, dtype=np.float32)
    assert np.array_equal(b.download(np.float32), np.arange(1024, dtype=np.float32))
    v = b.slice_view(1024, 16)
    assert v.byte_offset() == 1024 and v.byte_len() == 64
    assert np.array_equal(v.as_slice(np.float32), np.arange(256, 272, dtype=np.float32))
    c = b.clone()
    del b
    assert c.as_slice(np.float32)[5] == 5.0             # storage lives as long as any handle
    with pytest.raises(mx.InvalidArgument):
        c.slice_view(4000, 100)


def test_pool_reuse(ctx):
    d = ctx.device
    pool = mx.MlxBufferPool()
    a = pool.alloc(d, 3000, mx.DType.U8)
    assert a.byte_len() == 4096 and pool.in_use_count() == 1 and pool.free_count() == 0
    ptr = a.contents_ptr()
    del a
    pool.reset()
    assert pool.free_count() == 1 and pool.free_bytes() == 4096 and pool.in_use_count() == 0
    b = pool.alloc(d, 4000, mx.DType.F32)
    assert b.contents_ptr() == ptr and pool.free_count() == 0
    pool.release(b)
    assert pool.free_count() == 1
    pool.clear()
    assert pool.free_count() == 0
    pool.register_existing(d, d.alloc_buffer(16, mx.DType.U8))


def test_session_equals_direct_dispatch_and_counters(ctx):
    d = ctx.device
    gtype, otype = TYPES["Q8_0"]
    n, k, m = 256, 1024, 2
    wq = normal_weights(1, n, k, otype)
    x = normal_acts(1, m, k)
    direct = ctx.matmul(gtype, wq, x, n, k)
    mx.reset_counters()
    ex = mx.GraphExecutor.new(d)
    s = ex.begin()
    inp, w = ctx.buf(x, mx.DType.F32), ctx.buf(wq, mx.DType.U8)
    out = d.alloc_buffer(m * n * 4, mx.DType.F32)
    s.quantized_matmul_ggml(ctx.registry, d, inp, w, out, mx.GgmlQuantizedMatmulParams(m, n, k, gtype))
    s.barrier()
    t = s.finish_with_gpu_time()
    assert np.array_equal(out.as_slice(np.float32).reshape(m, n), direct)
    assert mx.dispatch_count() == 1 and mx.kernel_launch_count() == 1 and mx.barrier_count() == 1
    assert mx.sync_count() == 1 and mx.cmd_buf_count() == 1 and 0 < t < 1.0
    # dropping an encoder without committing is safe
    s2 = ex.begin()
    s2.quantized_matmul_ggml(ctx.registry, d, inp, w, out, mx.GgmlQuantizedMatmulParams(m, n, k, gtype))
    del s2


def test_buffer_dropped_after_encode_stays_alive(ctx):
    d = ctx.device
    gtype, otype = TYPES["Q4_0"]
    n, k = 512, 2048
    wq = normal_weights(2, n, k, otype)
    x = normal_acts(2, 1, k)
    want = ctx.matmul(gtype, wq, x, n, k)
    enc = d.command_encoder()
    inp, w = ctx.buf(x, mx.DType.F32), ctx.buf(wq, mx.DType.U8)
    out = d.alloc_buffer(n * 4, mx.DType.F32)
    mx.quantized_matmul_ggml(enc, ctx.registry, d, inp, w, out, mx.GgmlQuantizedMatmulParams(1, n, k, gtype))
    del inp, w                                   # the encoder holds them until the wait returns
    enc.commit()
    enc.wait_until_completed()
    assert np.array_equal(out.as_slice(np.float32), want[0])


def test_capture_and_replay(ctx):
    d = ctx.device
    gtype, otype = TYPES["Q6_K"]
    n, k = 1024, 4096
    wq = normal_weights(3, n, k, otype)
    w = ctx.buf(wq, mx.DType.U8)
    inp = ctx.buf(normal_acts(3, 1, k), mx.DType.F32)
    out = d.alloc_buffer(n * 4, mx.DType.F32)
    p = mx.GgmlQuantizedMatmulParams(1, n, k, gtype)
    enc = d.command_encoder()
    mx.quantized_matmul_ggml(enc, ctx.registry, d, inp, w, out, p)   # uploads happen outside the capture
    enc.commit_and_wait()
    first = out.as_slice(np.float32).copy()
    mx.reset_counters()
    enc.begin_capture()
    for _ in range(4):
        mx.quantized_matmul_ggml(enc, ctx.registry, d, inp, w, out, p)
    graph = enc.end_capture()
    assert mx.kernel_launch_count() == 0         # recording does not run anything
    graph.launch(enc)
    graph.launch(enc)
    enc.commit_and_wait()
    assert mx.kernel_launch_count() == 8 and mx.dispatch_count() == 8
    assert np.array_equal(out.as_slice(np.float32), first)


def test_wrap_external_device_memory(ctx):
    torch = pytest.importorskip("torch")
    d = ctx.device
    gtype, otype = TYPES["Q8_0"]
    n, k = 128, 512
    wq = normal_weights(4, n, k, otype)
    x = normal_acts(4, 1, k)
    tw = torch.from_numpy(wq).cuda()
    tx = torch.from_numpy(x).cuda()
    ty = torch.zeros(n, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    enc = d.command_encoder()
    mx.quantized_matmul_ggml(enc, ctx.registry, d, d.wrap_device_memory(tx.data_ptr(), x.nbytes, mx.DType.F32),
                             d.wrap_device_memory(tw.data_ptr(), wq.nbytes, mx.DType.U8),
                             d.wrap_device_memory(ty.data_ptr(), n * 4, mx.DType.F32),
                             mx.GgmlQuantizedMatmulParams(1, n, k, gtype))
    enc.commit_and_wait()
    y_ref, _ = orc.qmatmul(otype, wq, x, n, k)
    assert np.allclose(ty.cpu().numpy(), y_ref[0], rtol=1e-4, atol=1e-5)


# ---- concurrent groups: operations without buffer conflicts may overlap (the reference dispatches concurrently
# ---- and orders dependent dispatches with memory barriers, src/encoder.rs:837-853, src/graph.rs:1494-1530)
@pytest.mark.parametrize("qmv", ["auto", "stream"])
@pytest.mark.parametrize("captured", [False, True])
def test_dependent_chain_and_independent_ops_in_one_encoder(ctx, qmv, captured):
    mx.set_option("qmv", qmv)
    d = ctx.device
    gtype, otype = TYPES["Q8_0"]
    m, k, n1, n2 = 4, 1024, 2048, 512
    w1, w2, w3 = normal_weights(21, n1, k, otype), normal_weights(22, n2, n1, otype), normal_weights(23, n2, k, otype)
    x = normal_acts(21, m, k)
    xb, w1b, w2b, w3b = (ctx.buf(x, mx.DType.F32), ctx.buf(w1, mx.DType.U8), ctx.buf(w2, mx.DType.U8),
                         ctx.buf(w3, mx.DType.U8))
    y1 = d.alloc_buffer(m * n1 * 4, mx.DType.F32)
    y2 = d.alloc_buffer(m * n2 * 4, mx.DType.F32)
    y3 = d.alloc_buffer(m * n2 * 4, mx.DType.F32)
    p1 = mx.GgmlQuantizedMatmulParams(m, n1, k, gtype)
    p2 = mx.GgmlQuantizedMatmulParams(m, n2, n1, gtype)
    p3 = mx.GgmlQuantizedMatmulParams(m, n2, k, gtype)
    enc = d.command_encoder()

    def encode():
        mx.quantized_matmul_ggml(enc, ctx.registry, d, xb, w1b, y1, p1)   # y1 = x W1^T
        mx.quantized_matmul_ggml(enc, ctx.registry, d, xb, w3b, y3, p3)   # independent of the first: other lane
        mx.quantized_matmul_ggml(enc, ctx.registry, d, y1, w2b, y2, p2)   # reads y1: ordered after the first
        mx.quantized_matmul_ggml(enc, ctx.registry, d, xb, w3b, y3, p3)   # writes y3 again: ordered after the second

    if captured:
        encode()
        enc.commit_and_wait()
        enc.begin_capture()
        encode()
        g = enc.end_capture()
        for _ in range(3):
            g.launch(enc)
        enc.commit_and_wait()
    else:
        for _ in range(3):
            encode()
        enc.commit_and_wait()
    r1, ad1 = orc.qmatmul(otype, w1, x, n1, k, nthreads=8)
    got1 = y1.as_slice(np.float32).reshape(m, n1)
    assert norm_err(got1, r1, ad1) <= MV_TOL
    r2, ad2 = orc.qmatmul(otype, w2, got1.copy(), n2, n1, nthreads=8)
    assert norm_err(y2.as_slice(np.float32).reshape(m, n2), r2, ad2) <= MV_TOL
    r3, ad3 = orc.qmatmul(otype, w3, x, n2, k, nthreads=8)
    assert norm_err(y3.as_slice(np.float32).reshape(m, n2), r3, ad3) <= MV_TOL


def test_graph_replay_with_host_views(ctx):
    """An input written through its host view before the capture is uploaded by the graph at every replay, and an
    output with a host view is fetched back by the commit after each replay (unified-memory behaviour upstream)."""
    d = ctx.device
    gtype, otype = TYPES["Q8_0"]
    n, k, m = 512, 1024, 2
    wq = normal_weights(41, n, k, otype)
    w = ctx.buf(wq, mx.DType.U8)
    xb = d.alloc_buffer(m * k * 4, mx.DType.F32)
    yb = d.alloc_buffer(m * n * 4, mx.DType.F32)
    yb.as_slice(np.float32)                                  # give the output a host view
    p = mx.GgmlQuantizedMatmulParams(m, n, k, gtype)
    enc = d.command_encoder()
    x0 = normal_acts(41, m, k)
    xb.as_mut_slice(np.float32)[:] = x0.reshape(-1)
    mx.quantized_matmul_ggml(enc, ctx.registry, d, xb, w, yb, p)
    enc.commit_and_wait()
    xb.as_mut_slice(np.float32)[:] = x0.reshape(-1)          # dirty again: the capture records the upload
    enc.begin_capture()
    mx.quantized_matmul_ggml(enc, ctx.registry, d, xb, w, yb, p)
    g = enc.end_capture()
    for seed in (42, 43, 44):
        x = normal_acts(seed, m, k)
        xb.as_mut_slice(np.float32)[:] = x.reshape(-1)
        g.launch(enc)
        enc.commit_and_wait()
        y_ref, ad = orc.qmatmul(otype, wq, x, n, k, nthreads=8)
        assert norm_err(yb.as_slice(np.float32).reshape(m, n), y_ref, ad) <= MV_TOL


def test_graph_outlives_eager_growth_of_the_encoder_scratch(ctx):
    """A captured graph owns the scratch arenas its kernels address: a larger eager operation on the same encoder
    afterwards (which outgrows and hands back the encoder's own arena) must not disturb a later replay."""
    mx.set_option("qmv", "tc")                               # the mat-vec kernel that uses scratch memory
    d = ctx.device
    gtype, otype = TYPES["Q8_0"]
    n, k, m = 512, 1024, 4
    wq = normal_weights(51, n, k, otype)
    x = normal_acts(51, m, k)
    w, xb = ctx.buf(wq, mx.DType.U8), ctx.buf(x, mx.DType.F32)
    yb = d.alloc_buffer(m * n * 4, mx.DType.F32)
    p = mx.GgmlQuantizedMatmulParams(m, n, k, gtype)
    enc = d.command_encoder()
    mx.quantized_matmul_ggml(enc, ctx.registry, d, xb, w, yb, p)
    enc.commit_and_wait()
    enc.begin_capture()
    mx.quantized_matmul_ggml(enc, ctx.registry, d, xb, w, yb, p)
    g = enc.end_capture()
    assert mx.last_kernel_name() == "qmv_tc"
    # a prefill-sized mat-mat on the same encoder: its packed activations need a much larger arena
    n2, k2, m2 = 256, 4096, 512
    w2q = normal_weights(52, n2, k2, otype)
    x2 = normal_acts(52, m2, k2)
    y2 = ctx.matmul(gtype, w2q, x2, n2, k2)
    w2, x2b = ctx.buf(w2q, mx.DType.U8), ctx.buf(x2, mx.DType.F32)
    y2b = d.alloc_buffer(m2 * n2 * 4, mx.DType.F32)
    mx.quantized_matmul_ggml(enc, ctx.registry, d, x2b, w2, y2b, mx.GgmlQuantizedMatmulParams(m2, n2, k2, gtype))
    enc.commit_and_wait()
    assert np.array_equal(y2b.as_slice(np.float32).reshape(m2, n2), y2)
    yb.as_mut_slice(np.float32)[:] = 0
    g.launch(enc)
    enc.commit_and_wait()
    y_ref, ad = orc.qmatmul(otype, wq, x, n, k, nthreads=8)
    assert norm_err(yb.as_slice(np.float32).reshape(m, n), y_ref, ad) <= MV_TOL
    # a graph replays on the encoder that recorded it
    other = d.command_encoder()
    other_is_same = False
    try:
        g.launch(other)
        other_is_same = True     # a pooled encoder may hand the recording encoder's resources out again
    except mx.InvalidArgument as e:
        assert "encoder that recorded it" in str(e)
    if other_is_same:
        other.commit_and_wait()
    mx.set_option("qmv", "auto")


def test_host_view_rewritten_right_after_a_replay(ctx):
    """The replay's upload node reads the pinned host view when the stream gets there; a host write issued straight
    after graph_launch (no wait) has to wait for that read instead of changing what the replay sees."""
    d = ctx.device
    gtype, otype = TYPES["Q8_0"]
    n, k, m = 2048, 4096, 1
    wq = normal_weights(61, n, k, otype)
    w = ctx.buf(wq, mx.DType.U8)
    xb = d.alloc_buffer(m * k * 4, mx.DType.F32)
    ys = [d.alloc_buffer(m * n * 4, mx.DType.F32) for _ in range(2)]
    p = mx.GgmlQuantizedMatmulParams(m, n, k, gtype)
    enc = d.command_encoder()
    xs = [normal_acts(61 + i, m, k) for i in range(3)]
    graphs = []
    for yb in ys:
        xb.as_mut_slice(np.float32)[:] = xs[0].reshape(-1)
        mx.quantized_matmul_ggml(enc, ctx.registry, d, xb, w, yb, p)
        enc.commit_and_wait()
        xb.as_mut_slice(np.float32)[:] = xs[0].reshape(-1)
        enc.begin_capture()
        mx.quantized_matmul_ggml(enc, ctx.registry, d, xb, w, yb, p)
        graphs.append(enc.end_capture())
    xb.as_mut_slice(np.float32)[:] = xs[1].reshape(-1)
    graphs[0].launch(enc)
    xb.as_mut_slice(np.float32)[:] = xs[2].reshape(-1)       # no wait in between
    graphs[1].launch(enc)
    enc.commit_and_wait()
    for yb, x in zip(ys, xs[1:]):
        y_ref, ad = orc.qmatmul(otype, wq, x, n, k, nthreads=8)
        assert norm_err(yb.as_slice(np.float32).reshape(m, n), y_ref, ad) <= MV_TOL


def test_bounded_wait_that_runs_out_is_reported_and_recoverable(ctx):
    """src/encoder.rs:1867-1878, src/error.rs:87-89: a failed command buffer surfaces as CommandBufferError at the wait
    and is transient.  Here the failure is a kernel wait that gives up after its limit; nothing faults or hangs, the
    kernel returns normally with a status word, and the same encoder computes correctly afterwards."""
    d = ctx.device
    gtype, otype = TYPES["Q8_0"]
    n, k, m = 256, 1024, 2
    wq = normal_weights(71, n, k, otype)
    x = normal_acts(71, m, k)
    enc = d.command_encoder()
    enc.debug_wait_probe(1000)
    with pytest.raises(mx.CommandBufferError, match="gave up waiting for data") as ei:
        enc.commit_and_wait()
    assert ei.value.is_transient()
    w, xb = ctx.buf(wq, mx.DType.U8), ctx.buf(x, mx.DType.F32)
    yb = d.alloc_buffer(m * n * 4, mx.DType.F32)
    mx.quantized_matmul_ggml(enc, ctx.registry, d, xb, w, yb, mx.GgmlQuantizedMatmulParams(m, n, k, gtype))
    enc.commit_and_wait()                                    # the status word was cleared: no stale error
    y_ref, ad = orc.qmatmul(otype, wq, x, n, k, nthreads=8)
    assert norm_err(yb.as_slice(np.float32).reshape(m, n), y_ref, ad) <= MV_TOL
    with pytest.raises(mx.InvalidArgument):
        enc.debug_wait_probe(0)


def test_pool_alloc_batch_and_labeled_commits(ctx):
    d = ctx.device
    pool = mx.MlxBufferPool()
    bufs = pool.alloc_batch(d, [(3000, mx.DType.U8, [3000]), (64, mx.DType.F32, [4, 4]), (5000, mx.DType.F32, None)])
    assert [b.byte_len() for b in bufs] == [4096, 64, 8192] and bufs[1].shape() == [4, 4]
    assert pool.in_use_count() == 3
    with pytest.raises(mx.InvalidArgument):
        pool.alloc_batch(d, [(128, mx.DType.U8, None), (0, mx.DType.U8, None)])
    assert pool.in_use_count() == 3                          # all or nothing: the first request of the failed batch went back
    enc = d.command_encoder()
    gtype, otype = TYPES["Q4_0"]
    wq = normal_weights(81, 64, 256, otype)
    w, xb = ctx.buf(wq, mx.DType.U8), ctx.buf(normal_acts(81, 1, 256), mx.DType.F32)
    yb = d.alloc_buffer(64 * 4, mx.DType.F32)
    mx.quantized_matmul_ggml(enc, ctx.registry, d, xb, w, yb, mx.GgmlQuantizedMatmulParams(1, 64, 256, gtype))
    enc.commit_labeled("layer.test")
    enc.wait_until_completed()
    mx.quantized_matmul_ggml(enc, ctx.registry, d, xb, w, yb, mx.GgmlQuantizedMatmulParams(1, 64, 256, gtype))
    enc.commit_and_wait_labeled("layer.test")
    n_cb, ns = mx.profile_cb_get("layer.test")
    assert (n_cb, ns) == (0, 0) or ns > 0                    # the table fills only under MLX_PROFILE_CB=1


def test_peer_barrier_passes_when_everyone_arrived_and_gives_up_otherwise(ctx):
    """The library's cross-rank barrier on one GPU: two "ranks" whose flag arrays are ordinary buffers here.  With the
    other rank's arrival already in place the barrier passes; without it the bounded wait runs out, the commit reports
    CommandBufferError (transient) and the encoder keeps working.  Nothing hangs: the kernel returns by itself."""
    d = ctx.device
    mine = d.alloc_buffer(32 * 4, mx.DType.U32)
    theirs = d.alloc_buffer(32 * 4, mx.DType.U32)
    ptrs = [mine.contents_ptr(), theirs.contents_ptr()]          # rank 0 = this process
    enc = d.command_encoder()
    # rank 1 "arrived" at epoch 1: its flag in rank 0's array (slot 1) is set
    flags = np.zeros(32, np.uint32)
    flags[1] = 1
    mine.upload(flags)
    mx.peer_barrier(enc, 0, 2, ptrs, 1, limit_us=200000)
    enc.commit_and_wait()
    assert theirs.download(np.uint32)[0] == 1                    # this rank's arrival was published to the other one
    assert mine.download(np.uint32)[0] == 1                      # and to itself
    # epoch 2: nobody else arrives
    mx.peer_barrier(enc, 0, 2, ptrs, 2, limit_us=2000)
    with pytest.raises(mx.CommandBufferError, match="another rank") as ei:
        enc.commit_and_wait()
    assert ei.value.is_transient()
    mx.peer_barrier(enc, 0, 1, ptrs[:1], 3, limit_us=2000)       # a one-rank group never waits
    enc.commit_and_wait()
    with pytest.raises(mx.InvalidArgument):
        mx.peer_barrier(enc, 2, 2, ptrs, 1)


# ---- conflict tracking is by byte range: operations on views of one storage that do not overlap are independent
def test_views_of_one_arena_do_not_conflict(ctx):
    from oracle import oracle as orc
    from tests.gpu_util import MV_TOL, TYPES, norm_err, normal_acts, normal_weights
    gtype, otype = TYPES["Q8_0"]
    d = ctx.device
    mx.set_option("qmv", "auto")
    n, k, cnt = 512, 1024, 4
    ws = [normal_weights(40 + i, n, k, otype) for i in range(cnt)]
    xs = normal_acts(40, cnt, k)
    xin = d.alloc_buffer(cnt * k * 4, mx.DType.F32)
    yout = d.alloc_buffer(cnt * n * 4, mx.DType.F32)
    xin.as_mut_slice(np.float32)[:] = xs.reshape(-1)              # one host write, one upload
    xv = [xin.slice_view(i * k * 4, k) for i in range(cnt)]
    yv = [yout.slice_view(i * n * 4, n) for i in range(cnt)]
    p = mx.GgmlQuantizedMatmulParams(1, n, k, gtype)
    wb = [ctx.buf(w, mx.DType.U8) for w in ws]
    mx.reset_counters()
    enc = d.command_encoder()
    for i in range(cnt):
        mx.quantized_matmul_ggml(enc, ctx.registry, d, xv[i], wb[i], yv[i], p)
    enc.commit_and_wait()
    assert mx.kernel_launch_count() == 1                           # four mat-vecs, disjoint views: one batched launch
    y = yout.as_slice(np.float32).reshape(cnt, n)
    for i in range(cnt):
        y_ref, ad = orc.qmatmul(otype, ws[i], xs[i][None], n, k)
        assert norm_err(y[i][None], y_ref, ad) <= MV_TOL
    # overlapping views do conflict: the second call reads what the first one writes (its input view covers y row 0)
    mx.reset_counters()
    enc = d.command_encoder()
    mx.quantized_matmul_ggml(enc, ctx.registry, d, xv[0], wb[0], yv[0], p)
    y0_as_input = yout.slice_view(0, k)                            # the first k floats of the arena = rows 0 and 1 of y
    mx.quantized_matmul_ggml(enc, ctx.registry, d, y0_as_input, wb[1], yv[3], p)
    enc.commit_and_wait()
    assert mx.kernel_launch_count() == 2
    x2 = yout.as_slice(np.float32)[:k].copy()
    y_ref, ad = orc.qmatmul(otype, ws[1], x2[None], n, k)
    assert norm_err(yout.as_slice(np.float32).reshape(cnt, n)[3][None], y_ref, ad) <= MV_TOL
