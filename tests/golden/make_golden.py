"""Regenerates the golden fixtures in this directory from a checkout of the reference.

Usage:  python tests/golden/make_golden.py /path/to/reference

Needs the reference checkout (it is read as data: numeric tables are parsed out of its source
text, and the PEFT fixture is pushed through the same torch expression its offline parity script
uses).  The outputs are committed; the tests never read the reference itself.

  e4m3_lut.json        the 256-entry E4M3 -> FP32 table of kernels/gb10/common/e4m3_lut.cuh:22-88
  e2m1_lut.json        the 16-entry E2M1 table of kernels/gb10/common/dequant_nvfp4_bf16.cu:26-29
  peft_delta_k_proj.npz  lora_A / lora_B of layer 11 k_proj from test_data/lora-holo-tiny and
                       delta = scaling * B.float() @ A.float() (scripts/reference_deltas.py:77-93),
                       first 32 input columns
  peft_holo_tiny_pairs.npz  for every (layer, module) pair of that adapter: its PEFT key, the shapes, and of
                       delta = scaling * B @ A (float64 accumulation of the BF16 factors) the sum, the sum of magnitudes
                       and the top-left 4 x 4 block
"""
import json
import os
import re
import sys

import numpy as np

if len(sys.argv) < 2:
    sys.exit(__doc__)
REF = sys.argv[1]
OUT = os.path.dirname(os.path.abspath(__file__))


def floats_in_braces(text: str):
    body = text[text.index("{") + 1: text.index("};")]
    body = re.sub(r"//[^\n]*", "", body)
    return [float(tok.rstrip("f")) for tok in re.findall(r"-?\d+\.?\d*(?:[eE][-+]?\d+)?f", body)]


def main():
    src = open(os.path.join(REF, "kernels/gb10/common/e4m3_lut.cuh")).read()
    lut = floats_in_braces(src[src.index("E4M3_LUT[256]"):])
    assert len(lut) == 256
    # keep the sign of zero: -0.0f entries are emitted as "-0.0"
    json.dump([repr(v) for v in lut], open(os.path.join(OUT, "e4m3_lut.json"), "w"))

    src = open(os.path.join(REF, "kernels/gb10/common/dequant_nvfp4_bf16.cu")).read()
    e2m1 = floats_in_braces(src[src.index("DQ_E2M1_LUT[16]"):])
    assert len(e2m1) == 16
    json.dump([repr(v) for v in e2m1], open(os.path.join(OUT, "e2m1_lut.json"), "w"))

    import torch
    from safetensors.torch import load_file
    d = os.path.join(REF, "test_data/lora-holo-tiny")
    cfg = json.load(open(os.path.join(d, "adapter_config.json")))
    r, alpha, rs = int(cfg["r"]), float(cfg["lora_alpha"]), bool(cfg["use_rslora"])
    scaling = alpha / (r ** 0.5) if rs else alpha / r
    t = load_file(os.path.join(d, "adapter_model.safetensors"))
    key = "base_model.model.model.language_model.layers.11.self_attn.k_proj"
    a, b = t[key + ".lora_A.weight"], t[key + ".lora_B.weight"]
    delta = scaling * (b.float() @ a.float())
    np.savez_compressed(
        os.path.join(OUT, "peft_delta_k_proj.npz"),
        a_bits=a.view(torch.int16).numpy().view(np.uint16), b_bits=b.view(torch.int16).numpy().view(np.uint16),
        scaling=np.float32(scaling), r=np.int32(r), alpha=np.float32(alpha), use_rslora=np.int32(rs),
        delta_cols32=delta[:, :32].contiguous().numpy())
    keys = sorted(k[: -len(".lora_A.weight")] for k in t if k.endswith(".lora_A.weight"))
    sums, abs_sums, corners, shapes = [], [], [], []
    for k in keys:
        a64 = t[k + ".lora_A.weight"].double().numpy()
        b64 = t[k + ".lora_B.weight"].double().numpy()
        dl = scaling * (b64 @ a64)
        sums.append(dl.sum()); abs_sums.append(np.abs(dl).sum()); corners.append(dl[:4, :4].copy())
        shapes.append([b64.shape[0], a64.shape[1], a64.shape[0]])
    np.savez_compressed(os.path.join(OUT, "peft_holo_tiny_pairs.npz"), keys=np.array(keys), sums=np.array(sums),
                        abs_sums=np.array(abs_sums), corners=np.array(corners), shapes=np.array(shapes, dtype=np.int64),
                        n_tensors=np.int64(len(t)), scaling=np.float64(scaling))
    print("wrote", os.listdir(OUT))


if __name__ == "__main__":
    main()
