"""Generate the committed golden vectors under tests/golden/ (run in a container that has the
reference tree and the gguf python package; the outputs travel, the reference does not).

    python tests/golden/make_golden.py [/path/to/reference]

Writes
  routing.json          the reference's own routing function `_lcpp_op`
                        (plugin/vllm_gguf_plugin/quantization/linear.py:85-114), imported and evaluated
                        on a grid of (rows n, type, weight rows, K, packed) that covers every boundary
                        its test pins (tests/cpu/test_lcpp_routing.py:14-60)
  dequant_blocks.npz    seeded synthetic blocks of the four in-scope types and gguf-py's
                        `gguf.quants.dequantize` of them (the third-party reference decoder the
                        reference pins against llama.cpp, tests/cpu/test_dequant_fixtures.py:54-64)
  fixture_check.json    for each of the reference's real-row fixtures of the four types
                        (tests/fixtures/dequant/*.npz): sha256 of the raw bytes, of the stored gguf-py
                        output, and whether oracle.blocks.dequantize reproduced it bit for bit when
                        this script ran
  dequant_blocks_f1.npz, fixture_check_f1.json
                        the same two for the six low-bit types of the model file (Q2_K, IQ2_XXS, IQ2_XS,
                        IQ2_S, IQ3_XXS, IQ1_M) and oracle.blocks_f1
  iq3_ref_packed.npz    a seeded IQ3_S weight (64 rows x 1024 columns) and the reference's own load-time
                        repack of it (plugin/vllm_gguf_plugin/quantization/iq3_pack.py:134-138), the
                        input its packed kernels read; lets a GPU box run those kernels without the
                        reference tree. Also records that the reference's unpack(pack(w)) == w.
"""

import hashlib
import json
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "vllm-gsqrco-exl3_b200"))


def import_reference_linear(ref):
    """Import quantization/linear.py without running the plugin's package __init__ (which needs a newer
    huggingface_hub than this image has): stub the two parent packages with their real __path__."""
    plug = os.path.join(ref, "plugin", "vllm_gguf_plugin")
    for name, path in (("vllm_gguf_plugin", plug), ("vllm_gguf_plugin.quantization", os.path.join(plug, "quantization"))):
        m = types.ModuleType(name)
        m.__path__ = [path]
        sys.modules[name] = m
    import importlib

    return importlib.import_module("vllm_gguf_plugin.quantization.linear")


def routing(ref):
    lin = import_reference_linear(ref)
    types_ = [10, 12, 14, 16, 17, 18, 21, 22, 23, 29]
    ns = [1, 2, 3, 4, 5, 6, 7, 8, 9, 12, 16, 17, 24, 32, 33, 48, 64, 128, 2048]
    shapes = [(1024, 5120), (2048, 5120), (2049, 5120), (5120, 5120), (12032, 5120), (12288, 5120), (17408, 5120),
              (5120, 17408), (6144, 10240), (151936, 5120)]
    cases = []
    for t in types_:
        for n in ns:
            for rows, k in shapes:
                for packed in (False, True):
                    cases.append([n, t, rows, k, packed, lin._lcpp_op(n, t, rows, k, packed)])
    const = {
        "_OWN_QUANTIZE_OPS": list(lin._OWN_QUANTIZE_OPS), "_X_DTYPE_OPS": list(lin._X_DTYPE_OPS),
        "PACKED_VEC_MAX_ROWS": lin.PACKED_VEC_MAX_ROWS, "_FP32_DST_BUDGET": lin._FP32_DST_BUDGET,
    }
    with open(os.path.join(HERE, "routing.json"), "w") as f:
        json.dump({"source": "plugin/vllm_gguf_plugin/quantization/linear.py::_lcpp_op", "constants": const,
                   "columns": ["n", "type", "rows", "k", "packed", "op"], "cases": cases}, f)
    print("routing.json:", len(cases), "cases")


def dequant_blocks():
    import gguf
    from gguf import quants

    from gsq_b200 import synth

    out = {}
    for name, t in synth.TYPE_IDS.items():
        raw = synth.make_weight(t, 4, 512, 4242 + t)
        out[f"{name}_raw"] = raw
        out[f"{name}_ref"] = quants.dequantize(raw, gguf.GGMLQuantizationType(t)).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "dequant_blocks.npz"), **out)
    print("dequant_blocks.npz written; gguf", getattr(gguf, "__version__", "?"))


def dequant_blocks_f1():
    import gguf
    from gguf import quants

    from gsq_b200 import synth

    out = {}
    for name, t in synth.LOW_BIT_TYPE_IDS.items():
        raw = synth.make_weight(t, 4, 512, 4242 + t)
        out[f"{name}_raw"] = raw
        out[f"{name}_ref"] = quants.dequantize(raw, gguf.GGMLQuantizationType(t)).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "dequant_blocks_f1.npz"), **out)
    print("dequant_blocks_f1.npz written")


def fixture_check_f1(ref):
    from oracle import blocks_f1

    import glob

    rec = []
    for f in sorted(glob.glob(os.path.join(ref, "tests", "fixtures", "dequant", "*.npz"))):
        z = np.load(f)
        t = int(z["ggml_type"])
        if t not in blocks_f1.BLOCK_BYTES:
            continue
        mine = blocks_f1.dequantize(z["raw"], t)[0]
        rec.append({"file": os.path.basename(f), "type": t,
                    "raw_sha256": hashlib.sha256(np.ascontiguousarray(z["raw"]).tobytes()).hexdigest(),
                    "ref_sha256": hashlib.sha256(np.ascontiguousarray(z["ref"]).tobytes()).hexdigest(),
                    "oracle_bit_exact": bool(np.array_equal(mine.view(np.uint32), z["ref"].view(np.uint32)))})
    with open(os.path.join(HERE, "fixture_check_f1.json"), "w") as fo:
        json.dump({"source": "tests/fixtures/dequant/*.npz", "fixtures": rec}, fo, indent=1)
    print("fixture_check_f1.json:", len(rec), "fixtures,", sum(r["oracle_bit_exact"] for r in rec), "bit exact")


def fixture_check(ref):
    from oracle import blocks

    d = os.path.join(ref, "tests", "fixtures", "dequant")
    rec = []
    for f in sorted(os.listdir(d)):
        if not f.endswith(".npz"):
            continue
        z = np.load(os.path.join(d, f))
        t = int(z["ggml_type"])
        if t not in blocks.BLOCK_BYTES:
            continue
        mine = blocks.dequantize(z["raw"], t)[0]
        rec.append({
            "file": f, "type": t, "k": int(z["ref"].shape[0]),
            "raw_sha256": hashlib.sha256(z["raw"].tobytes()).hexdigest(),
            "ref_sha256": hashlib.sha256(z["ref"].tobytes()).hexdigest(),
            "oracle_bit_exact": bool(np.array_equal(mine.view(np.uint32), z["ref"].view(np.uint32))),
        })
    with open(os.path.join(HERE, "fixture_check.json"), "w") as fo:
        json.dump({"source": "tests/fixtures/dequant/*.npz", "fixtures": rec}, fo, indent=1)
    print("fixture_check.json:", sum(r["oracle_bit_exact"] for r in rec), "of", len(rec), "bit exact")


def iq3_ref_packed(ref):
    import importlib

    import torch

    from gsq_b200 import synth

    import_reference_linear(ref)        # installs the package stubs
    rp = importlib.import_module("vllm_gguf_plugin.quantization.iq3_pack")
    raw = synth.make_weight(21, 64, 1024, 77)
    w = torch.from_numpy(raw.copy())
    packed = rp.pack(w, 21)
    assert torch.equal(rp.unpack(packed, 21), w)
    np.savez_compressed(os.path.join(HERE, "iq3_ref_packed.npz"), raw=raw, ref_packed=packed.numpy(), seed=77)
    print("iq3_ref_packed.npz:", raw.shape, "round trip ok")


if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ["GSQ_REFERENCE"]
    dequant_blocks()
    fixture_check(ref)
    dequant_blocks_f1()
    fixture_check_f1(ref)
    routing(ref)
    iq3_ref_packed(ref)
