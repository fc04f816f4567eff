"""The all-gather folded into the stores of the config-5 kernels, and the CUDA-IPC buffers it writes into.

One GPU is enough for both: the ranks' gathered tensors are emulated by separate buffers of the one device (a peer pointer is
just another address to the kernel), and the IPC mapping is exercised by a second process on the same GPU."""
import multiprocessing as mp
import os
import sys

import numpy as np
import pytest

import oracle as O
from gpu_util import dev, empty, host, ulp16_diff

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 3, 8])
def test_gathered_kernels_fill_every_ranks_tensor(world):
    import puter_b200

    O.build()
    d = puter_b200.Device()
    rows, C, I, dt = 16, 1024, 1536, O.BF16
    T = world * rows
    rng = np.random.default_rng(world)
    mk = lambda *s: O.from_f32(rng.standard_normal(s).astype(np.float32), dt)
    x, r, br, gate, up = mk(T, C), mk(T, C), mk(T, C), mk(T, I), mk(T, I)
    gamma = O.from_f32(rng.uniform(0.5, 1.5, C).astype(np.float32), dt)
    mod = O.from_f32(rng.uniform(0, 1, (world, 3 * C)).astype(np.float32), dt)  # one batch item per rank
    h = O.binary(O.ADD, dt, x, r)
    want_n = O.rmsnorm(dt, h, gamma, 1e-6)
    want_g = O.gated_residual(dt, h, br, mod, T, C, rows, 3 * C, 0).reshape(T, C)
    want_s = O.gated_tensors(O.SWIGLU, dt, gate, up)
    n_all = [empty(T * C * 2) for _ in range(world)]
    g_all = [empty(T * C * 2) for _ in range(world)]
    s_all = [empty(T * I * 2) for _ in range(world)]
    cfg = puter_b200.RMSNormConfig(1e-6)
    for rank in range(world):
        sl = slice(rank * rows, (rank + 1) * rows)
        d.AddRMSNormGatedResidualGather(cfg, dev(x[sl]), dev(r[sl]), dev(gamma), dev(br[sl]), dev(mod[rank:rank + 1]), n_all, g_all, world, rank,
                                        rows, C, rows, 3 * C, 0, dt)
        d.SwiGLUTensorsGather(s_all, world, rank, dev(gate[sl]), dev(up[sl]), rows * I, dt)
    for rank in range(world):
        assert np.array_equal(host(g_all[rank], np.uint16, (T, C)), want_g)
        assert ulp16_diff(host(n_all[rank], np.uint16, (T, C)), want_n).max() <= 1
        assert ulp16_diff(host(s_all[rank], np.uint16, (T, I)), want_s).max() <= 1
        # every rank's copy is the same bits (one kernel wrote them all)
        assert np.array_equal(host(n_all[rank], np.uint16), host(n_all[0], np.uint16))
        assert np.array_equal(host(s_all[rank], np.uint16), host(s_all[0], np.uint16))
    with pytest.raises(puter_b200.DeviceError):  # more ranks than the kernels carry peer slots for
        d.SwiGLUTensorsGather(s_all * 9, 9 * world, 0, dev(gate[:rows]), dev(up[:rows]), rows * I, dt)
    assert d.take_error() == 0


def _child(handle, nbytes, conn):
    sys.path.insert(0, ROOT)
    import torch

    import puter_b200

    d = puter_b200.Device(0)
    buf = d.open_shared(handle, nbytes)
    t = torch.as_tensor(buf, device="cuda")
    seen = t[:8].cpu().tolist()
    t[8:16] = torch.arange(100, 108, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    buf.close()
    conn.send(seen)
    conn.close()


def test_shared_buffer_is_visible_to_a_second_process():
    import torch

    import puter_b200

    d = puter_b200.Device()
    buf = d.alloc_shared(4096)
    t = torch.as_tensor(buf, device="cuda")
    t.zero_()
    t[:8] = torch.arange(1, 9, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    ctx = mp.get_context("spawn")
    parent, child = ctx.Pipe()
    p = ctx.Process(target=_child, args=(buf.handle, buf.nbytes, child))
    p.start()
    seen = parent.recv()
    p.join(120)
    assert p.exitcode == 0
    assert seen == list(range(1, 9))
    assert t[8:16].cpu().tolist() == list(range(100, 108))
    with pytest.raises(puter_b200.DeviceError):  # only the library's own allocations can be exported
        wrapped = d._ref(torch.zeros(16, dtype=torch.uint8, device="cuda"))
        d._check(d.lib.cuda_buffer_ipc_export(wrapped, bytes(64), None))
    buf.close()
