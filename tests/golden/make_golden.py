"""Generates the golden fixtures under tests/golden/ by IMPORTING the reference's own Python tooling
(tools/extract_weights.py, tools/qat_golden_loader.py) from the reference tree.  Run it only where that tree
exists (it does not travel to the GPU box); the .npz files it writes are committed.

    python tests/golden/make_golden.py [/path/to/reference]

rtn_q4.npz  quantize_int4() of seeded float weights: the on-disk packed int4 bytes and fp32 scales
            (tools/extract_weights.py:124-140) -> pins oracle_pack_q4 and the nibble order.
dequant.npz dequant_chunks() of a packed file with fp32 and fp16 scales (tools/qat_golden_loader.py:29-47)
            -> pins the weight decode w = (nibble - 8) * scale, low nibble = even index.
"""
import os
import sys
import tempfile
from pathlib import Path

import numpy as np

here = os.path.dirname(os.path.abspath(__file__))
# the reference checkout: first argument, else W4A8_REFERENCE_DIR, else a directory "reference" beside this repository
ref = sys.argv[1] if len(sys.argv) > 1 else (os.environ.get("W4A8_REFERENCE_DIR") or
                                             os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(here))), "reference"))
sys.path.insert(0, os.path.join(ref, "tools"))
import extract_weights as ew          # noqa: E402
import qat_golden_loader as qgl       # noqa: E402

rng = np.random.default_rng(31)
w = rng.normal(size=(12, 160)).astype(np.float32) * 0.05
w[0, :32] = 0.0                       # an all-zero block: scale 1e-8, nibbles 8
w[3, 64:96] *= 40.0                   # a block with a large range
w[5, 7] = 0.35                        # lone outlier
packed, scale = ew.quantize_int4(w)
np.savez(os.path.join(here, "rtn_q4.npz"), w=w, packed=packed, scale=scale)

with tempfile.TemporaryDirectory() as td:
    q, s32, s16 = Path(td) / "q.bin", Path(td) / "s32.bin", Path(td) / "s16.bin"
    packed.tofile(q)
    scale.astype("<f4").tofile(s32)
    scale.astype("<f2").tofile(s16)
    d32 = np.concatenate([np.asarray(b[1], dtype=np.float32).ravel() for b in qgl.dequant_chunks(q, s32, 0)])
    d16 = np.concatenate([np.asarray(b[1], dtype=np.float32).ravel() for b in qgl.dequant_chunks(q, s16, 1)])
np.savez(os.path.join(here, "dequant.npz"), packed=packed, scale=scale, dequant_fp32_scale=d32, dequant_fp16_scale=d16)
print("wrote", sorted(f for f in os.listdir(here) if f.endswith(".npz")))
