"""Generates tests/golden/packer_mse_scale.npz with the REFERENCE packer's own MSE row-scale search
(choose_mse_int8_weight_scale, reference tools/difflux2sample.cpp:1225-1259) through
oracle/_ref/difpacker_scale, which oracle/Makefile builds from the reference checkout by including
the tool's source file. Rows: what the packer hands that function -- rotated weight rows -- plus
the edge cases (all zero, one outlier, tiny and huge magnitudes, widths 256 / 768 / 4096). And whole
runs of the packer itself (rewrite_named_linear_w8a8, :1607-2096) on small bf16 weights: the codes,
scales and input-equalisation vectors of the cache files it wrote.

Run it where that checkout is present:  python tests/golden/make_packer_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

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


PACK_CASES = [(2, 16, 512, True, True), (3, 16, 512, False, True), (5, 16, 256, True, False), (6, 16, 256, True, True),
              (4, 4, 4096, True, True), (7, 4, 4096, False, False)]  # implementation, N, K, equalise, mse


def pack_weight(impl, N, K):
    rng = np.random.default_rng(7000 + impl)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    w[:, rng.integers(0, K, 5)] *= 12.0
    w[1] = 0.0
    w[2, 9] = 1.5
    return ob.f32_to_bf16(w)


def main():
    import tempfile
    from diffusion_compiler_b200 import convrot_cache
    data = {}
    for name, rows in cases().items():
        data[name + "/rows"] = rows
        data[name + "/scale_bits"] = ob.packer_mse_scales(rows).view(np.uint32)
    # whole packer runs (rewrite_named_linear_w8a8): weight in, the cache file's tensors out
    for impl, N, K, equalise, mse in PACK_CASES:
        w = pack_weight(impl, N, K)
        with tempfile.TemporaryDirectory() as d:
            with convrot_cache.Cache(ob.packer_pack(w, impl, equalise, mse, d)) as cache:
                key = "pack_impl%d_eq%d_mse%d" % (impl, equalise, mse)
                data[key + "/weight"] = w
                data[key + "/codes"] = cache.tensor("weight")[1].view(np.int8).copy()
                data[key + "/scale_bits"] = cache.tensor("scale")[1].view(np.uint32).copy()
                if equalise:
                    data[key + "/input_scale"] = cache.tensor("input_scale")[1].view(np.uint16).copy()
    np.savez_compressed(os.path.join(HERE, "packer_mse_scale.npz"), **data)
    print("wrote", len(data), "arrays")


if __name__ == "__main__":
    main()
