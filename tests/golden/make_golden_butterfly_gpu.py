"""Butterfly fixtures produced by the REFERENCE'S OWN GPU kernels (needs a CUDA device + Triton).

The butterfly product of the reference lives in a third-party CUDA op that is not available
offline, and the reference has no pure-PyTorch butterfly; the only executable statement of its
stage / stride / twiddle-index convention is its Triton scan
(src/gru_qat/triton_kernels/scan_butterfly.py:369-459 forward, 971-1075 backward).  This script
runs exactly those two wrappers -- from the unmodified package that ``oracle/make_ref.py``
installs into ``oracle/_ref`` -- on a few tiny seeded problems and stores inputs and outputs.
They take the twiddle tensor directly and synchronise only inside a CTA, so they need neither
``torch_structured`` nor a grid-wide spin-wait.

The Triton kernels are accurate to about 3e-2 relative (README.md:187-198 of the reference), so
these fixtures pin the CONVENTION (a wrong stride order, twiddle axis or 2x2 orientation gives
O(1) errors), not the last digits; ``tests/test_oracle_golden.py`` compares the CPU oracle with
them at that tolerance.

    python tests/golden/make_golden_butterfly_gpu.py [output directory]
"""

from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)
sys.path.insert(0, os.path.join(REPO, "oracle", "_ref"))

from gru_qat.triton_kernels import scan_butterfly as ref_bfly  # noqa: E402
from oracle import gru_scan_oracle as orc  # noqa: E402  (seeded problem generator only)

# name, T, B, H, stacked factors, seed, quant
CASES = [
    ("ref_butterfly_h16", 4, 3, 16, 1, 11, None),
    ("ref_butterfly_h8_nb2", 3, 2, 8, 2, 12, None),          # odd factor index: reversed stride order
    ("ref_butterfly_h12_pad", 3, 5, 12, 1, 13, None),        # H = 12 padded to 16
    ("ref_butterfly_h32_nb2", 5, 9, 32, 2, 14, None),
    ("ref_butterfly_h16_q8", 4, 3, 16, 1, 15, ((0.02, -127, 127), (0.02, -127, 127))),
]


def main(out_dir: str) -> None:
    os.makedirs(out_dir, exist_ok=True)
    dev = torch.device("cuda")
    for name, T, B, H, nb, seed, quant in CASES:
        gi, h0, tw, bh, dout = orc.make_problem("butterfly", T, B, H, seed, butterfly_nblocks=nb)
        qi, qo = quant if quant else (None, None)
        g = [t.to(dev) for t in (gi, h0, tw, bh, dout)]
        out = ref_bfly.gru_scan_butterfly_forward_triton(g[0], g[1], g[2], g[3], h_in_quant=qi, h_out_quant=qo)
        dgi, dh0, dtw, dbh = ref_bfly.gru_scan_butterfly_backward_triton(
            g[0], g[1], g[2], g[3], out, g[4], h_in_quant=qi, h_out_quant=qo)
        torch.cuda.synchronize()
        q = lambda t: np.array([], dtype=np.float64) if t is None else np.array(t, dtype=np.float64)  # noqa: E731
        np.savez_compressed(os.path.join(out_dir, name + ".npz"),
                            gi=gi.numpy(), h0=h0.numpy(), W=tw.numpy(), bh=bh.numpy(), dout=dout.numpy(),
                            out=out.cpu().numpy(), dgi=dgi.cpu().numpy(), dh0=dh0.cpu().numpy(),
                            dW=dtw.cpu().numpy(), dbh=dbh.cpu().numpy(), q_in=q(qi), q_out=q(qo))
        print(f"wrote {name}: out max {out.abs().max().item():.4f}", flush=True)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
