"""Measurement kernels of the library, run from the command line (a B200 is needed):

    python -m qwental_b200.probes stream    # what a ring of bulk (TMA) copies pulls out of HBM: the staging mechanism alone
    python -m qwental_b200.probes umma      # issue rate of tcgen05 MMAs of M = 128, K = 16 for several N

Both print one line per configuration.  Times are CUDA-event times of the launch (qw_batch_end).
"""
from __future__ import annotations

import struct
import sys

import numpy as np

from .gpu import Gpu
from .layers import u32


def stream(gpu: Gpu, sm: int = 148):
    k = gpu.compile("stream_probe", "stream_probe")
    sink = gpu.buf(4).zero()
    src = gpu.buf(sm * 34816 * 800)  # 4.1 GB: far more than L2

    def run(stage, nst, read, stride, mult):
        total = sm * stage * mult
        args = struct.pack("<QIIII", total, stage, nst, read, stride)

        def go():
            return gpu.batch().kernel(k).buf(0, src).buf(1, sink).bytes(2, args).dispatch((1,), (544,)).end() * 1e3

        go()
        go()
        ms = min(go() for _ in range(5))
        print("stage %6d B x %2d stages  read %d  strided %d  total %.2f GB  %8.1f us  %7.1f GB/s" % (stage, nst, read, stride, total / 1e9, ms * 1e3, total / ms / 1e6))

    for stage, nst in ((34816, 4), (34816, 6), (17408, 8), (8704, 16), (69632, 3)):
        for read in (0, 1):
            run(stage, nst, read, 0, (800 * 34816) // stage)
    for mult in (44, 90):  # the sizes of one expert-FFN launch and of one attention launch of the benchmark
        run(34816, 4, 1, 0, mult)


def umma(gpu: Gpu):
    k = gpu.compile("umma_bench", "umma_bench")
    out = gpu.buf(16).zero()
    for a_tmem in (1, 0):
        for n in (16, 32, 64, 128, 256):
            for nacc in (1, 4):
                if nacc * n > 256:
                    continue
                for _ in range(2):
                    gpu.batch().kernel(k).buf(0, out).bytes(1, u32(64, nacc, n, a_tmem)).dispatch((1,), (128,)).end()
                d = out.download(np.uint64, 2)
                print("A in %s  N %3d  accumulators %d  cycles per MMA %.1f (issue loop %.1f)" % ("tensor memory" if a_tmem else "shared memory", n, nacc, int(d[0]) / 1024, int(d[1]) / 1024))


def main(argv):
    if len(argv) != 2 or argv[1] not in ("stream", "umma"):
        sys.stderr.write(__doc__)
        return 2
    gpu = Gpu()
    try:
        (stream if argv[1] == "stream" else umma)(gpu)
    finally:
        gpu.close()
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
