"""Regenerates the committed golden fixtures from the reference tree.

Run where the reference tree is checked out and oracle/_ref has been built (make -C oracle):

    python tests/golden/make_golden.py /path/to/reference

Outputs (all small, committed):
  e4m3_codec_all_bf16.npz   the reference's fp8_e4m3::pack and NVIDIA's host
                            E4M3 / E5M2 SATFINITE conversion applied to every one
                            of the 65,536 bf16 bit patterns, plus unpack of all
                            256 codes
  e4m3_probe_kat.json       the inputs and pinned byte codes of
                            tests/fp8_e4m3_probe.cu:23-27,55-56
  moe_router_parity.json    the routing and expert-bank vectors of
                            tests/fixtures/moe_router_parity/{weights,unpacked_case}.json
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from oracle_bindings import RefHost  # noqa: E402


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("CANOPY_REFERENCE")
    if not ref_root or not os.path.isdir(ref_root):
        raise SystemExit("usage: make_golden.py /path/to/reference   (or set CANOPY_REFERENCE)")
    r = RefHost()
    allbf = (np.arange(65536, dtype=np.uint32) << 16).view(np.float32)
    unpack = np.array([r.lib.ref_e4m3_unpack(b) for b in range(256)], dtype=np.float32)
    np.savez_compressed(
        os.path.join(HERE, "e4m3_codec_all_bf16.npz"),
        ref_pack=r.pack_array(allbf),
        nv_e4m3=r.nv_array(allbf, False),
        nv_e5m2=r.nv_array(allbf, True),
        ref_unpack_bits=unpack.view(np.uint32),
    )

    # tests/fp8_e4m3_probe.cu:23-27 input list, :55-56 pinned codes (index -> byte).
    kat_inputs = [0.0, -0.0, 1.0, -1.0, 0.015625, 448.0, -448.0, 447.0, float("nan"), float("inf"), float("-inf")]
    bits = [int(np.float32(v).view(np.uint32)) for v in kat_inputs]
    packed = [int(b) for b in r.pack_array(np.array(kat_inputs, dtype=np.float32))]
    with open(os.path.join(HERE, "e4m3_probe_kat.json"), "w") as f:
        json.dump({"input_f32_bits": bits, "ref_pack": packed,
                   "pinned": {"1": 0x80, "5": 0x7e, "6": 0xfe, "8": 0x7f, "9": 0x7f}}, f, indent=1)

    fx = os.path.join(ref_root, "tests", "fixtures", "moe_router_parity")
    w = json.load(open(os.path.join(fx, "weights.json")))
    u = json.load(open(os.path.join(fx, "unpacked_case.json")))
    keep_w = ["H", "num_experts", "top_k", "TRUNK_I", "EXPERT_I", "trunk_fc_in_w", "trunk_fc_out_w",
              "expert_fc_in_w", "expert_fc_out_w"]
    keep_u = ["logits", "route_weights_pre_inhibition", "route_weights", "hidden_gated", "mixed"]
    with open(os.path.join(HERE, "moe_router_parity.json"), "w") as f:
        json.dump({**{k: w[k] for k in keep_w}, **{k: u[k] for k in keep_u}}, f)


if __name__ == "__main__":
    main()
