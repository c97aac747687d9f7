"""Bounded waits that run out, on the GPU: a wait for a flag that nothing sets returns after its poll limit, records its
error code in the status word the host reads, leaves the context usable and the next launch of the same kernel clean.
Nothing here hangs or faults: every wait has a limit of a few thousand polls."""
import ctypes

import pytest
import torch

from owl_engine_b200.ops import gemm_tc, kernels as K
from owl_engine_b200.parallel import symm as SY

pytestmark = pytest.mark.gpu
DEV = "cuda"
WAIT_PEER = 3


def test_peer_wait_runs_out_and_reports():
    SY.SymmetricWorkspace.status()                      # clear
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    res = torch.full((1,), -7, dtype=torch.int32, device=DEV)
    K.call("owl_comm_wait_probe", K.ptr(flag), 5, 3000, K.ptr(res), K.stream())
    torch.cuda.synchronize()
    assert int(res.item()) == WAIT_PEER
    assert SY.SymmetricWorkspace.status() == WAIT_PEER
    assert SY.SymmetricWorkspace.status() == 0          # reading clears the word
    flag.fill_(5)                                       # the flag is there: the same wait passes at once
    K.call("owl_comm_wait_probe", K.ptr(flag), 5, 3000, K.ptr(res), K.stream())
    torch.cuda.synchronize()
    assert int(res.item()) == 0 and SY.SymmetricWorkspace.status() == 0


def test_all_gather_gated_gemm_unwinds_when_its_tiles_never_arrive():
    """The column-parallel GEMM waits per row tile for the all-gather's sequence flag. In a world of one with a sequence
    number nobody publishes the producer's wait runs out: the kernel must drain its pipeline, free its tensor memory and
    report, and the next (satisfied) launch must give the right product."""
    t, n, hdim = 256, 512, 1024
    pipe = SY.PrefillPipe.local(hdim, t, DEV)
    g = torch.Generator(device=DEV).manual_seed(0)
    x = (torch.randn(t, hdim, device=DEV, generator=g) * 0.5).half()
    w = (torch.randn(n, hdim, device=DEV, generator=g) * 0.05).half()
    pipe.x(t, torch.float16).copy_(x)
    out = torch.zeros(t, n, dtype=torch.bfloat16, device=DEV)
    gemm_tc.gemm_status()
    K.call("owl_f16_gemm_ag", K.ptr(pipe.x(t, torch.float16)), hdim, K.ptr(w), hdim, K.ptr(out), t, n, hdim, n, 0,
           K.ptr(pipe.ag_flags), 7, 1, pipe.max_local, 2000, K.stream())          # flags are 0, 7 never comes
    torch.cuda.synchronize()                                                        # returns: nothing hangs
    assert gemm_tc.gemm_status() == WAIT_PEER
    assert gemm_tc.gemm_status() == 0
    pipe.ag_flags.fill_(7)
    K.call("owl_f16_gemm_ag", K.ptr(pipe.x(t, torch.float16)), hdim, K.ptr(w), hdim, K.ptr(out), t, n, hdim, n, 0,
           K.ptr(pipe.ag_flags), 7, 1, pipe.max_local, 2000, K.stream())
    torch.cuda.synchronize()
    assert gemm_tc.gemm_status() == 0
    want = x.float() @ w.float().t()
    err = (out.float() - want).norm() / want.norm()
    assert err < 1e-2, err
    # tensor memory was released by the aborted launch: a plain GEMM of the same shape still runs
    out2 = torch.zeros_like(out)
    gemm_tc.f16_gemm(x, w, out2)
    torch.cuda.synchronize()
    assert ((out2.float() - want).norm() / want.norm()) < 1e-2


def test_status_words_are_all_readable_and_clean():
    st = K.all_status()
    assert set(st) == {"skinny", "fma", "stream_tc", "gemm", "gemm_dense", "gemm_nvfp4", "attn_tc", "comm"} and not any(st.values()), st
