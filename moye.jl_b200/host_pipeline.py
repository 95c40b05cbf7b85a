"""Host-to-host GEMM steps with the PCIe copies hidden behind the kernel.

`matmul(A, B, C)` of the reference takes device arrays (examples/gemm.jl:66-89); a caller whose
operands live in host memory has to copy them in and the result out.  Doing the three phases of
every step back to back on one stream leaves the GPU idle during the copies.  `HostGemmPipeline`
runs host->device copies, the GEMM and the device->host copy on three streams over a small ring of
device buffers, so step i+1's operands travel while step i multiplies and step i-1's result
drains.  Every step still moves all of its own bytes.
"""
import torch

from .algorithm import plan_gemm
from .array import MoYeArray

__all__ = ["HostGemmPipeline"]


class HostGemmPipeline:
    def __init__(self, M, N, K, in_dtype, out_dtype, device=None, depth=2, comm=None, **gemm_kw):
        """`comm` (a `Communicator`) makes B a replicated operand of several ranks: only rank 0 copies it from the
        host, the others receive it over NVLink (`moye_b200_bcast`), which takes N - 1 copies of B off the PCIe links."""
        self.comm = comm
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.depth = depth
        d = self.device
        self.A = [torch.empty(M, K, dtype=in_dtype, device=d) for _ in range(depth)]
        self.B = [torch.empty(N, K, dtype=in_dtype, device=d) for _ in range(depth)]
        self.C = [torch.empty(M, N, dtype=out_dtype, device=d) for _ in range(depth)]
        self.plans = [plan_gemm(MoYeArray(c), MoYeArray(a), MoYeArray(b), None, **gemm_kw)
                      for a, b, c in zip(self.A, self.B, self.C)]
        self.s_in, self.s_mm, self.s_out = (torch.cuda.Stream(d) for _ in range(3))
        self.mm_ptr = self.s_mm.cuda_stream
        self.in_ready = [torch.cuda.Event() for _ in range(depth)]
        self.mm_done = [torch.cuda.Event() for _ in range(depth)]
        self.out_done = [torch.cuda.Event() for _ in range(depth)]
        self.count = 0
        self.h2d_bytes = self.A[0].numel() * self.A[0].element_size() + self.B[0].numel() * self.B[0].element_size()
        self.d2h_bytes = self.C[0].numel() * self.C[0].element_size()

    def start_after(self, event):
        """Make all three streams wait for `event` (e.g. the start marker of a timed region)."""
        for s in (self.s_in, self.s_mm, self.s_out):
            s.wait_event(event)

    def submit(self, A_host, B_host, C_host):
        """Queue one step: pinned host A (M,K), B (N,K) in, pinned host C (M,N) out."""
        import ctypes
        k = self.count % self.depth
        reuse = self.count >= self.depth
        with torch.cuda.stream(self.s_in):
            if reuse:
                self.s_in.wait_event(self.mm_done[k])     # the GEMM that last read A[k], B[k] has finished
            self.A[k].copy_(A_host, non_blocking=True)
            if self.comm is None or self.comm.rank == 0:
                self.B[k].copy_(B_host, non_blocking=True)
            if self.comm is not None:
                self.comm.bcast(self.B[k], 0, stream=ctypes.c_void_p(self.s_in.cuda_stream))
            self.in_ready[k].record(self.s_in)
        self.s_mm.wait_event(self.in_ready[k])
        if reuse:
            self.s_mm.wait_event(self.out_done[k])        # C[k] of the previous round has left the device
        self.plans[k](ctypes.c_void_p(self.mm_ptr))
        self.mm_done[k].record(self.s_mm)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.mm_done[k])
            C_host.copy_(self.C[k], non_blocking=True)
            self.out_done[k].record(self.s_out)
        self.count += 1

    def join(self, stream=None):
        """Make `stream` (default: the current stream) wait for everything submitted so far."""
        stream = stream or torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_mm, self.s_out):
            ev = torch.cuda.Event()
            ev.record(s)
            stream.wait_event(ev)
