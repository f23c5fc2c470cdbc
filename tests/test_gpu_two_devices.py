"""Two contexts on two GPUs of one process: the launch set-up of the radix-32 FFT passes (opt-in shared-memory size,
resident-CTA count, SM count) is per device. Skipped on a box that shows one GPU. Own kernels only, no peer memory."""
import numpy as np
import pytest

from test_gpu_ops import up_cols
from util import edge_m31_column

pytestmark = pytest.mark.gpu


def test_fft_on_second_device_of_one_process(zkb, oracle):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    ctxs = [zkb.Context(device=d, max_log_size=16) for d in (0, 1)]
    try:
        for log_n, log_out in ((13, 15), (14, 14)):
            for c in ctxs:  # device 0 first, then device 1: the second must not reuse the first's set-up
                vals = np.stack([edge_m31_column(900 + k, 1 << log_n) for k in range(3)])
                bufs, ptrs = up_cols(c, vals)
                c.ifft_cols(ptrs, log_n)
                coeffs = oracle.interpolate_cols(vals, log_n)
                assert (np.stack([b.download() for b in bufs]) == coeffs).all()
                outs = [c.alloc(1 << log_out) for _ in range(3)]
                c.lde_cols(ptrs, log_n, [o.ptr for o in outs], log_out)
                assert (np.stack([o.download() for o in outs]) == oracle.evaluate_cols(coeffs, log_n, log_out)).all()
    finally:
        for c in ctxs:
            c.close()
