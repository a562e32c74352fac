"""Two independent host-buffer calls side by side.

``SpMMbase.run_host`` / ``SDDMMbase.run_host`` are synchronous: upload, launch, download,
wait.  Back to back, the host link idles while one call computes and the GPU idles while the
other one's result travels.  When the two calls do not depend on each other (the SpMM and the
SDDMM of one GNN layer read the same features) they can be issued from two host threads on
two CUDA streams, so that one call's transfers overlap the other's kernels and the link
carries uploads and downloads at the same time (PCIe is full duplex).  The C-ABI host
entry points release the interpreter lock while they wait, which is what lets two Python
threads do this.
"""
import threading
import time

import torch


class HostPair(object):
    """Runs ``spmm.run_host(x_host, y_host)`` and ``sddmm.run_host(src_host, dst_host,
    out_host)`` concurrently, each on its own stream; ``run`` returns when both results are
    in host memory.  Single-GPU modules only (the sharded operators issue collectives, which
    must be enqueued in the same order on every rank)."""

    def __init__(self, spmm, sddmm):
        self.spmm, self.sddmm = spmm, sddmm
        self.device = spmm.ctx.torch_device
        self.streams = (torch.cuda.Stream(device=self.device),
                        torch.cuda.Stream(device=self.device))

    def _call(self, which, fn, args, errors, delay=0.0):
        try:
            if delay:
                time.sleep(delay)
            torch.cuda.set_device(self.device)
            with torch.cuda.stream(self.streams[which]):
                fn(*args)
        except BaseException as exc:        # handed to the caller's thread
            errors.append(exc)

    def run(self, x_host, y_host, src_host, dst_host, out_host):
        main = torch.cuda.current_stream(self.device)
        for s in self.streams:
            s.wait_stream(main)
        errors = []
        # The SDDMM call is the longer chain (two uploads, then a result of 4 bytes per edge to
        # bring back), so it is issued from this thread, at once: its uploads reach the copy
        # engine ahead of the SpMM's, whose thread holds its call back for a moment.
        t = threading.Thread(target=self._call,
                             args=(0, self.spmm.run_host, (x_host, y_host), errors, 3e-4))
        t.start()
        self._call(1, self.sddmm.run_host, (src_host, dst_host, out_host), errors)
        t.join()
        for s in self.streams:
            main.wait_stream(s)
        if errors:
            raise errors[0]
        return y_host, out_host
