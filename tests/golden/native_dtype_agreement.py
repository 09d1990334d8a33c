"""Secondary statistic of the parity contract: how often the reference's NATIVE 16-bit path agrees with the
fp32-upcast path that the CUDA encoder is bit-exact to.

Fed bf16 / fp16, the reference takes norms, codebook products, the similarity einsum and the threshold compare in
that dtype (src/quantizers/hqmq.py:127,136,157-158; outlier_aware.py:72), whose rounding depends on the backend,
so no kernel can match it bit for bit; the contract is "upcast to fp32, then exact".  This script measures, on
the reference itself (CPU), the share of 4-element chunks whose fake-quantised values are identical in both
paths once both are rounded to the 16-bit dtype.

    python tests/golden/native_dtype_agreement.py /path/to/reference
"""
import sys
import warnings

import torch

from make_golden import make_input


def main(ref_root):
    sys.path.insert(0, ref_root)
    warnings.filterwarnings("ignore")
    import hqmq  # the reference
    rows = []
    for name, S, br, C, shape, kind in [("s24_r3", 24, 3, None, (1, 4, 256, 128), "randn"),
                                         ("s96_r4+Med3x", 96, 4, 3.0, (2, 4, 256, 128), "hot"),
                                         ("s192_r6+Med3x", 192, 6, 3.0, (2, 2, 128, 128), "student")]:
        x = make_input(kind, shape, 77)
        for dt in (torch.bfloat16, torch.float16):
            q = hqmq.HQMQ(n_layers=1, n_heads=shape[1], secondary_size=S, radius_bits=br, device="cpu", seed=42)
            if C is not None:
                q = hqmq.with_outlier_extraction(q, C)
            xd = x.to(dt)
            with torch.no_grad():
                native = q.quantize_K(xd, 0)                       # arithmetic in dt
                upcast = q.quantize_K(xd.float(), 0).to(dt)        # the contract's path, rounded once at the end
            n = shape[3] // 4
            same = (native.view(*shape[:3], n, 4) == upcast.view(*shape[:3], n, 4)).all(-1)
            rel = float((native.float() - upcast.float()).norm() / upcast.float().norm())
            rows.append((name, str(dt).split(".")[-1], float(same.float().mean()), rel))
    for r in rows:
        print(f"{r[0]:16s} {r[1]:9s} identical chunks {100 * r[2]:6.2f} %   rel-L2 between the two paths {r[3]:.2e}")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: native_dtype_agreement.py /path/to/reference")
    main(sys.argv[1])
