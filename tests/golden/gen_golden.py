#!/usr/bin/env python3
"""Generate the golden vectors under tests/golden/ from the reference project.

Run in a checkout that has the reference project next to it:

    python tests/golden/gen_golden.py [--reference /path/to/reference]

It imports the reference's own Python quantizer/dequantizer
(Scripts/quantize/hq4.py, hq_blocks.py, pack.py), reads the reference's
committed test fixtures, and writes small .npz files plus one QWP1 pack that
the test-suite reads without the reference being present.  While generating it
also checks, bit for bit, that the C oracle (oracle/qw_oracle.c) agrees with
the reference on a larger random case than the committed fixtures hold.

Files written:
  ref_fixtures.npz   the reference's committed known-answer vectors, re-encoded:
                     selfpack blocks + dq4 (Tests/QWQuantTests/fixtures/selfpack.qwp[.dq4.npy]),
                     aq_quantizer_golden.json, aq_repack_golden.json,
                     fn_goldens.json["sparse_moe"].
  selfpack.qwp       pack_file() of the --selfpack tensor (Scripts/quantize/pack.py:742-758);
                     asserted byte-identical to the reference's committed fixture.
  formats.npz        quantize/dequantize outputs of the reference for HQ4_G32, HQ8_G32, HQ4_G64.
  moepack.qwp        pack_file() of a small layer: 3-D expert stacks ("….experts.…" names, Scripts/quantize/pack.py:104-112,
                     231-255) in HQ4_G32_M5, HQ8_G32 and HQ4_G64, plus 2-D HQ8_G32 / HQ4_G64 planes
  moepack.npz        the tensors that went into moepack.qwp and the reference's per-expert dequantised sidecars
  matmul.npz         reduced-size restatements of the fixture recipes of
                     Scripts/oracle/gen_s1_q4_fixtures.py, gen_f5_fixtures.py, gen_mlp_fixtures.py
                     (same seeds, distributions and arithmetic; smaller N/K).
"""
import argparse
import json
import os
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("QW_REFERENCE", os.path.join(os.path.dirname(str(ROOT)), "reference")))
    args = ap.parse_args()
    ref = Path(args.reference)
    sys.path.insert(0, str(ref / "Scripts" / "quantize"))
    import hq4  # noqa: E402  (reference module)
    import hq_blocks  # noqa: E402
    import pack  # noqa: E402
    from oracle import qw_oracle as qo

    qo.build(force=True)

    # ---- 1. the reference's committed known-answer vectors ------------------
    fx = ref / "Tests" / "QWQuantTests" / "fixtures"
    N, K = 256, 1024
    rr, cc = np.meshgrid(np.arange(N), np.arange(K), indexing="ij")
    w_self = (np.sin(rr * 0.013 + cc * 0.007) * 0.02).astype(np.float32)
    w_self[:, 5] *= np.float32(6.0)
    norm = np.sin(rr[:, 0] * 0.021) * 0.5 + 1.0
    with tempfile.TemporaryDirectory() as td:
        out = Path(td) / "selfpack.qwp"
        pack.pack_file({"w_test": w_self}, out, {"source": "selfpack", "sha256_source": "n/a"},
                       raw={"norm_test": norm})
        mine = out.read_bytes()
    theirs = (fx / "selfpack.qwp").read_bytes()
    assert mine == theirs, "regenerated selfpack.qwp differs from the reference's committed fixture"
    (HERE / "selfpack.qwp").write_bytes(mine)
    self_blocks = hq4.quant_hq4_g32_m5(w_self)
    dq4 = np.load(fx / "selfpack.qwp.dq4.npy")
    assert np.array_equal(hq4.dequant_hq4_g32_m5(self_blocks), dq4)
    raw_norm = np.load(fx / "selfpack.qwp.raw.npy")

    qg = json.loads((fx / "aq_quantizer_golden.json").read_text())
    rg = json.loads((fx / "aq_repack_golden.json").read_text())
    moe = json.loads((ref / "Tests" / "QWFlashNextTests" / "fixtures" / "fn_goldens.json").read_text())["sparse_moe"]

    def t(entry):
        return np.asarray(entry["data"], dtype=np.float32).reshape(entry["shape"])

    np.savez_compressed(
        HERE / "ref_fixtures.npz",
        selfpack_w=w_self, selfpack_blocks=self_blocks, selfpack_dq4=dq4, selfpack_raw_norm=raw_norm,
        aqq_bf16=np.frombuffer(bytes.fromhex(qg["bf16"]), dtype="<u2").reshape(qg["rows"], qg["cols"]),
        aqq_blocks=np.frombuffer(bytes.fromhex(qg["blocks"]), dtype=np.uint8).reshape(qg["rows"], qg["cols"] // 32, 20),
        repack_packed=np.frombuffer(bytes.fromhex(rg["packed"]), dtype=np.uint8).reshape(rg["rows"], -1),
        repack_codes=np.frombuffer(bytes.fromhex(rg["codes"]), dtype=np.uint8).reshape(rg["rows"], rg["cols"]),
        repack_scales=np.frombuffer(bytes.fromhex(rg["scales"]), dtype="<f4").reshape(rg["rows"], -1),
        repack_biases=np.frombuffer(bytes.fromhex(rg["biases"]), dtype="<f4").reshape(rg["rows"], -1),
        repack_values=np.frombuffer(bytes.fromhex(rg["values"]), dtype="<f4").reshape(rg["rows"], rg["cols"]),
        moe_cfg=np.asarray([moe["hidden"], moe["experts"], moe["top_k"], moe["expert_intermediate"],
                            moe["shared_intermediate"], int(moe["norm_topk_prob"])], dtype=np.int64),
        moe_gate=t(moe["weights"]["gate.weight"]),
        moe_gate_up=t(moe["weights"]["experts.gate_up_proj"]),
        moe_down=t(moe["weights"]["experts.down_proj"]),
        moe_sh_gate=t(moe["weights"]["shared_expert.gate_proj.weight"]),
        moe_sh_up=t(moe["weights"]["shared_expert.up_proj.weight"]),
        moe_sh_down=t(moe["weights"]["shared_expert.down_proj.weight"]),
        moe_sh_scalar=t(moe["weights"]["shared_expert_gate.weight"]),
        moe_input=t(moe["input"]), moe_output=t(moe["output"]),
    )

    # ---- 2. per-format quantize / dequantize outputs of the reference -------
    fmts = {"HQ4_G32": (4, 32, True), "HQ8_G32": (8, 32, False), "HQ4_G64": (4, 64, False)}
    rng = np.random.default_rng(20240)
    w_small = rng.normal(0.0, 0.02, (48, 256)).astype(np.float32)
    w_small[3, 64:96] = 0.0          # a zero-scale group
    w_small[5, 7] = 3.0              # an outlier
    w_small[7, 128:192] = 0.0125     # a constant (max == min) group
    arrays = {"w": w_small}
    for name, (bits, group, m5) in fmts.items():
        blocks, eff = hq_blocks.quant_hq_blocks(w_small, bits=bits, group=group, is_m5=m5)
        assert eff == group
        arrays[f"{name}_blocks"] = blocks
        arrays[f"{name}_rot"] = hq_blocks.dequant_hq_blocks_rot(blocks, bits, group, m5, f16_round=False)
        arrays[f"{name}_rot16"] = hq_blocks.dequant_hq_blocks_rot(blocks, bits, group, m5, f16_round=True)
        arrays[f"{name}_std"] = hq_blocks.dequant_hq_blocks(blocks, bits, group, m5)
    xs = rng.standard_normal((4, 256)).astype(np.float32)
    arrays["fwht_in"] = xs
    arrays["fwht_out"] = hq4.fwht32_ortho(xs)
    np.savez_compressed(HERE / "formats.npz", **arrays)

    # larger bit-exactness check of the C oracle against the reference (not stored)
    wl = np.random.default_rng(99).normal(0.0, 0.02, (512, 1024)).astype(np.float32)
    for name, (bits, group, m5) in fmts.items():
        fmt = qo.FORMATS[name]
        blocks, _ = hq_blocks.quant_hq_blocks(wl, bits=bits, group=group, is_m5=m5)
        mine = qo.quantize(wl, fmt)
        assert np.array_equal(mine, blocks), f"{name}: oracle quantizer differs from the reference"
        for f16r in (False, True):
            want = hq_blocks.dequant_hq_blocks_rot(blocks, bits, group, m5, f16_round=f16r)
            assert np.array_equal(qo.dequant(blocks, fmt, f16_round=f16r), want), name
        want = hq_blocks.dequant_hq_blocks(blocks, bits, group, m5)
        assert np.array_equal(qo.dequant(blocks, fmt, standard=True), want), name
    assert np.array_equal(qo.fwht32(wl), hq4.fwht32_ortho(wl))
    print("oracle == reference on 512x1024 for all formats (quantize, dequant rot/rot16/std, fwht)")

    # ---- 3. matmul fixtures: the reference's recipes at reduced size --------
    mm = {}
    # gen_s1_q4_fixtures.py: seed 7, x then W ~ U(-0.02, 0.02), y = wq @ f32(x)
    K = 640
    rng = np.random.default_rng(7)
    x = rng.uniform(-0.02, 0.02, size=K).astype(np.float32).astype(np.float16)
    for n in (32, 96):
        W = rng.uniform(-0.02, 0.02, size=(n, K)).astype(np.float32)
        blocks = hq4.quant_hq4_g32_m5(W)
        wq = hq4.dequant_hq4_g32_m5_rot(blocks, f16_round=True)
        mm[f"s1_N{n}_blocks"] = blocks
        mm[f"s1_N{n}_y"] = (wq @ x.astype(np.float32)).astype(np.float32)
    mm["s1_x"] = x
    # gen_f5_fixtures.py: seed 17, W ~ N(0, 1/sqrt(k)), M in {2,3,4,8}, x ~ N(0,1) f16
    rng = np.random.default_rng(17)
    for nm, (n, k) in {"f5a": (96, 512), "f5b": (40, 1280)}.items():
        W = (rng.standard_normal((n, k)) * (k ** -0.5)).astype(np.float32)
        blocks = hq4.quant_hq4_g32_m5(W)
        deq = hq4.dequant_hq4_g32_m5_rot(blocks, f16_round=True)
        mm[f"{nm}_blocks"] = blocks
        for M in (2, 3, 4, 8):
            xm = rng.standard_normal(k * M).astype(np.float32).astype(np.float16).reshape(M, k)
            mm[f"{nm}_x_M{M}"] = xm
            mm[f"{nm}_y_M{M}"] = np.einsum("nk,mk->mn", deq, xm.astype(np.float32), optimize=True).astype(np.float32)
    # gen_mlp_fixtures.py: seed 14, U(-0.02, 0.02) gate/up/down, x ~ N(0,1), h rounded to f16
    H, I = 256, 384
    rng = np.random.default_rng(14)
    gate = rng.uniform(-0.02, 0.02, size=(I, H)).astype(np.float32)
    up = rng.uniform(-0.02, 0.02, size=(I, H)).astype(np.float32)
    down = rng.uniform(-0.02, 0.02, size=(H, I)).astype(np.float32)
    gu_blocks = hq4.quant_hq4_g32_m5(np.concatenate([gate, up], axis=0))
    assert np.array_equal(gu_blocks[:I], hq4.quant_hq4_g32_m5(gate))
    dn_blocks = hq4.quant_hq4_g32_m5(down)
    pq = hq4.dequant_hq4_g32_m5_rot(gu_blocks, f16_round=True)
    dq = hq4.dequant_hq4_g32_m5_rot(dn_blocks, f16_round=True)
    mm["mlp_gu_blocks"] = gu_blocks
    mm["mlp_dn_blocks"] = dn_blocks
    for M in (1, 2, 8):
        xm = rng.standard_normal(size=(M, H)).astype(np.float32).astype(np.float16)
        xf = xm.astype(np.float32)
        hg = xf @ pq[:I].T
        hu = xf @ pq[I:].T
        h16 = (hg / (1.0 + np.exp(-hg)) * hu).astype(np.float16)
        mm[f"mlp_x_M{M}"] = xm
        mm[f"mlp_h_M{M}"] = h16
        mm[f"mlp_y_M{M}"] = (h16.astype(np.float32) @ dq.T).astype(np.float32)
    np.savez_compressed(HERE / "matmul.npz", **mm)

    # ---- 4. a pack with expert stacks and the rotated HQ containers --------
    rng = np.random.default_rng(31)
    stacks = {}
    # layer: (quant spec, experts, hidden, intermediate); weights are drawn as f16 values so that the .npz stays small
    layers = {"l0": (None, 4, 128, 128), "l1": ((8, 32, False), 4, 128, 128), "l2": ((4, 64, False), 2, 256, 256)}
    tensors = []

    def draw(shape, sigma):
        return rng.normal(0.0, sigma, shape).astype(np.float16)

    for layer, (kind, E, H, I) in layers.items():
        gu, dn = draw((E, 2 * I, H), 0.05), draw((E, H, I), 0.05)
        stacks[f"{layer}_gate_up"], stacks[f"{layer}_down"] = gu, dn
        for nm, arr in ((f"{layer}.mlp.experts.gate_up_proj", gu), (f"{layer}.mlp.experts.down_proj", dn)):
            arr = arr.astype(np.float32)
            tensors.append((nm, arr, kind) if kind else (nm, arr))
        stacks[f"{layer}_x"] = rng.standard_normal((24, H)).astype(np.float16)
        stacks[f"{layer}_logits"] = rng.standard_normal((24, E)).astype(np.float32)
    stacks["q_proj"], stacks["o_proj"] = draw((96, 128), 0.02), draw((64, 256), 0.02)
    tensors.append(("l0.attn.q_proj.weight", stacks["q_proj"].astype(np.float32), (8, 32, False)))
    tensors.append(("l0.attn.o_proj.weight", stacks["o_proj"].astype(np.float32), (4, 64, False)))
    with tempfile.TemporaryDirectory() as td:
        out = Path(td) / "moepack.qwp"
        pack.pack_file(tensors, out, {"source": "moepack", "sha256_source": "n/a"}, sidecar_dir=Path(td) / "side")
        (HERE / "moepack.qwp").write_bytes(out.read_bytes())
        for layer in layers:   # the reference's own dequantisation of expert 1 of each stack (first 16 rows)
            for proj in ("gate_up_proj", "down_proj"):
                stacks[f"{layer}_{proj}_e1_dq"] = np.load(Path(td) / "side" / f"{layer}.mlp.experts.{proj}.e1.dq4.npy")[:16]
    np.savez_compressed(HERE / "moepack.npz", **stacks)
    for f in ("ref_fixtures.npz", "selfpack.qwp", "formats.npz", "matmul.npz", "moepack.qwp", "moepack.npz"):
        print(f, (HERE / f).stat().st_size, "bytes")


if __name__ == "__main__":
    main()
