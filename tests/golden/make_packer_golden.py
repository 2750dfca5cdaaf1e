"""Generates tests/golden/packer_mse_scale.npz with the REFERENCE packer's own MSE row-scale search
(choose_mse_int8_weight_scale, reference tools/difflux2sample.cpp:1225-1259) through
oracle/_ref/difpacker_scale, which oracle/Makefile builds from the reference checkout by including
the tool's source file. Rows: what the packer hands that function -- rotated weight rows -- plus
the edge cases (all zero, one outlier, tiny and huge magnitudes, widths 256 / 768 / 4096).

Run it where that checkout is present:  python tests/golden/make_packer_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(os.path.dirname(HERE)))

import oracle_bridge as ob  # noqa: E402


def cases():
    rng = np.random.default_rng(20)
    out = {}
    for columns in (256, 768, 4096):
        rows = (rng.standard_normal((12, columns)) * 0.02).astype(np.float32)
        rows[1] = 0.0                                    # an all-zero output channel
        rows[2, 5] = 3.0                                 # one outlier: clipping pays
        rows[3] *= np.float32(1e-20)                     # tiny
        rows[4] *= np.float32(1e20)                      # huge
        rows[5] = rng.standard_t(2, columns).astype(np.float32)  # heavy tails
        rows[6] = np.round(rows[6] * 4096) / 4096        # few distinct values
        out["w%d" % columns] = rows
    return out


def main():
    data = {}
    for name, rows in cases().items():
        data[name + "/rows"] = rows
        data[name + "/scale_bits"] = ob.packer_mse_scales(rows).view(np.uint32)
    np.savez_compressed(os.path.join(HERE, "packer_mse_scale.npz"), **data)
    print("wrote", len(data), "arrays")


if __name__ == "__main__":
    main()
