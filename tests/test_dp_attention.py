"""Data-parallel attention + expert parallelism (parallel/dp_attention.py): two CPU ranks over gloo
against the single-rank model; the GPU forms of the exchange kernels, with the ranks played in turn on
one GPU, against the collective statement of the same exchange."""
import os
import subprocess
import sys

import pytest
import torch


def _torchrun(script, port, n=2, timeout=600, env=None):
    e = dict(os.environ, OMP_NUM_THREADS="2")
    e.update(env or {})
    return subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                           "--master-addr", "127.0.0.1", "--master-port", str(port), script],
                          capture_output=True, text=True, timeout=timeout, env=e)


def test_two_cpu_ranks_match_single_rank():
    res = _torchrun(os.path.join(os.path.dirname(__file__), "mp_dp_attention_worker.py"), 29557, env={"DP_WORKER_DEVICE": "cpu"})
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "DP_ATTENTION_OK" in res.stdout


def _bind():
    import ctypes as C
    from hartsyinference_b200.ops import _native as N
    vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_longlong, C.c_float
    return (N.bind("b200_dp_norm_gather", i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, f32, vp]),
            N.bind("b200_dp_gather_wait", i32, [vp, vp, vp, vp, vp, i32, i32, i32, i64, vp, vp]),
            N.bind("b200_dp_combine_scatter", i32, [vp, vp, vp, vp, i32, i32, vp, vp, vp, i32, i32, i32, i32, vp]),
            N.bind("b200_dp_reduce_norm", i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, f32, i64, vp, vp]))


def _table(tensors):
    import ctypes as C
    t = (C.c_void_p * 8)()
    for i, x in enumerate(tensors):
        t[i] = x.data_ptr()
    return t


def _rms(x, w, eps=1e-6):
    x = x.float()
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w.float()


@pytest.mark.gpu
@pytest.mark.parametrize("world,l,hidden,top_k", [(2, 3, 256, 2), (4, 8, 7168, 8), (8, 4, 2048, 0)])
def test_exchange_kernels_ranks_played_in_turn(world, l, hidden, top_k):
    """W ranks on one GPU, each kernel launched for all ranks before the next kernel (so every flag a
    kernel waits for was raised by a kernel that has finished), two calls in a row on the same buffers."""
    from hartsyinference_b200.ops import _native as N
    gather, wait, scatter, reduce = _bind()
    dev = torch.device("cuda")
    t = world * l
    gen = torch.Generator(device="cuda").manual_seed(1)
    bf = lambda *s: (torch.randn(*s, device=dev, generator=gen) * 0.5).to(torch.bfloat16)
    g = [torch.zeros(t, hidden, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    gl = [torch.zeros(t, 576, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    slots_buf = [torch.zeros(world, l, hidden, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    flags = [torch.zeros(16, dtype=torch.int32, device=dev) for _ in range(world)]
    ctr = [torch.zeros(8, dtype=torch.int32, device=dev) for _ in range(world)]
    caches = [torch.zeros(2 * t, 576, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    tg, tgl, ts, tf = _table(g), _table(gl), _table(slots_buf), _table(flags)
    res = [bf(l, hidden) for _ in range(world)]
    w1, w2 = bf(hidden).abs() + 0.5, bf(hidden).abs() + 0.5
    st = N.state(torch.device("cuda", torch.cuda.current_device())).status.data_ptr()
    for call in range(2):
        a = [bf(l, hidden) for _ in range(world)]
        slots_all = (torch.randperm(2 * t, device=dev, generator=gen)[:t]).to(torch.int64)
        slots_all[t - 1] = -1                                   # a padding row: nothing is stored for it
        for r in range(world):                                  # what the attention block wrote for the local rows
            own = slots_all[r * l:(r + 1) * l]
            caches[r][own[own >= 0]] = bf(int((own >= 0).sum()), 576)
        want_res = [(res[r].float() + a[r].float()).to(torch.bfloat16) for r in range(world)]
        want_g = torch.cat([_rms(want_res[r], w1) for r in range(world)])
        want_lat = torch.zeros(t, 576, device=dev)
        for r in range(world):
            for i in range(l):
                s = int(slots_all[r * l + i])
                if s >= 0:
                    want_lat[r * l + i] = caches[r][s].float()
        for r in range(world):
            assert gather(a[r].data_ptr(), res[r].data_ptr(), w1.data_ptr(), caches[r].data_ptr(),
                          slots_all[r * l:(r + 1) * l].contiguous().data_ptr(), tg, tgl, tf, ctr[r].data_ptr(), l, hidden, r, world,
                          1e-6, N.stream()) == 0
        for r in range(world):
            assert wait(gl[r].data_ptr(), caches[r].data_ptr(), slots_all.data_ptr(), flags[r].data_ptr(), ctr[r].data_ptr(), t, l, r,
                        100_000_000, st, N.stream()) == 0
        N.check_status()
        keep = slots_all >= 0
        for r in range(world):
            assert torch.equal(res[r], want_res[r])
            assert (g[r].float() - want_g).abs().max() < 0.02 * want_g.abs().max()
            assert torch.equal(caches[r][slots_all[keep]].float(), want_lat[keep])
        # ---- every rank's contribution to every row, combined and scattered to the owners
        n_slots = 64
        ys = [bf(n_slots, hidden) for _ in range(world)]
        shared = [bf(t, hidden) for _ in range(world)]
        slot_of = [torch.randint(-1, n_slots, (t, max(top_k, 1)), device=dev, generator=gen).to(torch.int32) for _ in range(world)]
        wts = [torch.rand(t, max(top_k, 1), device=dev, generator=gen) for _ in range(world)]
        part = []
        for r in range(world):
            acc = shared[r].float().clone()
            for k in range(top_k):
                hit = slot_of[r][:, k] >= 0
                acc[hit] += wts[r][hit, k, None] * ys[r][slot_of[r][hit, k].long()].float()
            part.append(acc.to(torch.bfloat16).float())
        for r in range(world):
            assert scatter(ys[r].data_ptr() if top_k else 0, slot_of[r].data_ptr() if top_k else 0, wts[r].data_ptr() if top_k else 0,
                           shared[r].data_ptr(), top_k, hidden, ts, tf, ctr[r].data_ptr(), t, l, r, world, N.stream()) == 0
        hs = [torch.empty(l, hidden, dtype=torch.bfloat16, device=dev) for _ in range(world)]
        for r in range(world):
            assert reduce(slots_buf[r].data_ptr(), res[r].data_ptr(), w2.data_ptr(), hs[r].data_ptr(), flags[r].data_ptr(),
                          ctr[r].data_ptr(), l, hidden, world, 1e-6, 100_000_000, st, N.stream()) == 0
        N.check_status()
        for r in range(world):
            tot = want_res[r].float() + sum(part[s][r * l:(r + 1) * l] for s in range(world))
            assert (res[r].float() - tot).abs().max() < 0.02 * tot.abs().max()
            ref = _rms(res[r], w2)
            assert (hs[r].float() - ref).abs().max() < 0.02 * ref.abs().max()
        assert all(int(c[0]) == call + 1 and int(c[4]) == call + 1 for c in ctr)


@pytest.mark.gpu
def test_missing_source_runs_out_and_reports():
    """Rank 0 of two runs alone: its waits for rank 1's rows give up after about a millisecond, the
    kernels return, the status word names the exchange; the context stays usable."""
    from hartsyinference_b200.exceptions import DeviceWaitTimeout
    from hartsyinference_b200.ops import _native as N
    gather, wait, scatter, reduce = _bind()
    dev = torch.device("cuda")
    world, l, hidden = 2, 2, 256
    t = world * l
    g = [torch.zeros(t, hidden, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    gl = [torch.zeros(t, 576, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    flags = [torch.zeros(16, dtype=torch.int32, device=dev) for _ in range(world)]
    ctr = torch.zeros(8, dtype=torch.int32, device=dev)
    res = torch.ones(l, hidden, dtype=torch.bfloat16, device=dev)
    w = torch.ones(hidden, dtype=torch.bfloat16, device=dev)
    slots = torch.full((t,), -1, dtype=torch.int64, device=dev)
    st = N.state(torch.device("cuda", torch.cuda.current_device())).status.data_ptr()
    assert gather(0, res.data_ptr(), w.data_ptr(), 0, slots.data_ptr(), _table(g), _table(gl), _table(flags), ctr.data_ptr(), l, hidden,
                  0, world, 1e-6, N.stream()) == 0
    assert wait(gl[0].data_ptr(), 0, slots.data_ptr(), flags[0].data_ptr(), ctr.data_ptr(), t, l, 0, 2_000_000, st, N.stream()) == 0
    with pytest.raises(DeviceWaitTimeout) as ei:
        N.check_status()
    assert ei.value.kernel == 12 and ei.value.site == 1
    h = torch.empty_like(res)
    slot_buf = torch.zeros(world, l, hidden, dtype=torch.bfloat16, device=dev)
    assert reduce(slot_buf.data_ptr(), res.data_ptr(), w.data_ptr(), h.data_ptr(), flags[0].data_ptr(), ctr.data_ptr(), l, hidden, world,
                  1e-6, 2_000_000, st, N.stream()) == 0
    with pytest.raises(DeviceWaitTimeout) as ei:
        N.check_status()
    assert ei.value.kernel == 12 and ei.value.site == 2
    assert torch.isfinite(h.float()).all()
    x = torch.randn(64, 64, device=dev)
    assert torch.isfinite(x @ x).all()


@pytest.mark.gpu
@pytest.mark.multigpu
def test_two_gpu_ranks_match_single_rank_collective_and_fused():
    res = _torchrun(os.path.join(os.path.dirname(__file__), "mp_dp_attention_worker.py"), 29558, env={"NCCL_NVLS_ENABLE": "0"})
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "DP_ATTENTION_OK" in res.stdout
