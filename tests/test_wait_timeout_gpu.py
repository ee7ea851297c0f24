"""A bounded wait that runs out: the kernel records it and returns, the context stays usable.

Every mbarrier wait of the kernels gives up after SPIO_WAIT_LIMIT_NS of wall time, sets the
CTA's abort flag and lets the kernel write a status word that ``spio_b200_device_status``
returns and clears (the reference reports driver errors as ``ValueError`` from
spio/cuda/driver.pyx:118-123; a wait that never ends would simply hang there).  The probe below
is a one-warp kernel built from the package's own ``ptx.cuh`` with the limit set to 0.2 ms; it
waits on a barrier nothing ever arrives on.  It returns by itself: no trap, no fault, no hang.
"""

import ctypes

import pytest
import torch

from oracle import oracle as O
from spio_b200 import _clib
from spio_b200.compiler import compile_kernel, load_kernel
from spio_b200.cuda import get_device_attributes
from tests import capi

pytestmark = pytest.mark.gpu

PROBE = r'''
#include "gw8_common.cuh"
using namespace spio_b200;
extern "C" __global__ void wait_probe(int* status, unsigned long long* waited_ns) {
  __shared__ __align__(8) u64 bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  volatile int* abortp = &abort_flag;
  const u64 t0 = globaltimer_ns();
  const bool ok = mbar_wait(smem_u32(&bar), 0u, abortp);  // nothing arrives: must give up
  const u64 t1 = globaltimer_ns();
  __syncthreads();
  if (threadIdx.x == 0) {
    *waited_ns = t1 - t0;
    if (!ok) atomicExch(status, (int)GW8_WAIT_TIMEOUT);
  }
}
'''


def test_a_wait_that_runs_out_is_reported_once_and_the_device_stays_usable():
    lib = _clib.load()
    assert capi.status() == 0
    arch = get_device_attributes(0).compute_capability
    cubin = compile_kernel(PROBE, source_name="wait_probe.cu", arch=arch,
                           defines={"SPIO_WAIT_LIMIT_NS": "200000ull"})
    module, fn = load_kernel("wait_probe", cubin, 0)
    address = ctypes.c_void_p()
    _clib.check(lib.spio_b200_status_address(ctypes.byref(address)))
    waited = torch.zeros(1, dtype=torch.int64, device="cuda:0")
    fn.launch(1, 32, [address, waited])
    torch.cuda.synchronize()
    assert 150_000 <= int(waited.item()) < 50_000_000      # gave up after the limit, not for ever
    assert capi.status() == 1                               # SPIO_STATUS_WAIT_TIMEOUT, reported ...
    assert capi.status() == 0                               # ... once
    module.unload()

    # the context is intact: the next convolution is correct
    sh = O.Shape(4, 64, 16, 16, 3, 3, 1, 1)
    x, w, b, dy = O.make_inputs(sh, seed=3, bias=True)
    xd, wd, bd = (capi.to_dev(t) for t in (x, w, b))
    O.assert_close(capi.fprop(xd, wd, bd, sh), O.c_fprop(x, w, b, sh), sh, "fprop", "after a timed-out wait")
    assert capi.status() == 0
