"""Generates tests/golden/ref_b200.npz: outputs of the REFERENCE's own kernels (cuda/nvfp4_ops.cu compiled
unmodified for sm_100a, oracle/_ref) run on a B200, for seeded inputs.

Run on a machine with a B200 and oracle/_ref built:   python tests/golden/make_golden.py [out.npz]
Operator-level vectors carry their inputs; the whole-block vectors carry the token rows, the routing and
the output, plus a hash of the synthetic layer they were computed on (the layer itself, 1.1 GB, is
regenerated from its seed by the tests).
"""
import hashlib
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

SEED, LAYER = 1234, 0


def u16(t):
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "ref_b200.npz")
    pkg = entry.load_package()
    pkg.load_library()
    from p92moe_b200 import synth

    orc = entry.load_oracle()
    ref = orc.ref()
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(2026)
    data = {}

    # router: logits (both orders) and top-8 on a seeded router weight
    router, bias = synth.make_router(SEED, LAYER)
    for rows in (1, 4):
        x = synth.make_activations(SEED, 100 + rows, rows)
        logits = torch.empty((rows, 256), dtype=torch.float32, device="cuda")
        if rows == 1:
            assert ref.ref_bf16_gemv_f32(x.data_ptr(), router.data_ptr(), logits.data_ptr(), 256, 2560, stream) == 0
        else:
            assert ref.ref_bf16_gemm_f32(x.data_ptr(), router.data_ptr(), logits.data_ptr(), rows, 256, 2560, stream) == 0
        ids = torch.empty((rows, 8), dtype=torch.int32, device="cuda")
        w = torch.empty((rows, 8), dtype=torch.float32, device="cuda")
        assert ref.ref_router_top8_rows(logits.data_ptr(), bias.data_ptr(), ids.data_ptr(), w.data_ptr(), rows, 2.5, stream) == 0
        data[f"router{rows}_x"] = u16(x)
        data[f"router{rows}_logits"] = logits.cpu().numpy()
        data[f"router{rows}_ids"] = ids.cpu().numpy()
        data[f"router{rows}_weights"] = w.cpu().numpy()
    data["router_w"] = u16(router)
    data["router_bias"] = bias.cpu().numpy()

    # quantiser, SwiGLU, combine, add
    xq_in = torch.empty((6, 1024), dtype=torch.float32, device="cuda").normal_(0, 1, generator=g).to(torch.bfloat16)
    xq_in[0, :16] = 0
    packed = torch.empty((6, 512), dtype=torch.uint8, device="cuda")
    scales = torch.empty((6, 64), dtype=torch.uint8, device="cuda")
    assert ref.ref_nvfp4_quantize(xq_in.data_ptr(), packed.data_ptr(), scales.data_ptr(), 6 * 1024, 1.0, stream) == 0
    data["quant_in"], data["quant_packed"], data["quant_scales"] = u16(xq_in), packed.cpu().numpy(), scales.cpu().numpy()
    gate = torch.empty(4096, dtype=torch.float32, device="cuda").normal_(0, 2, generator=g).to(torch.bfloat16)
    up = torch.empty(4096, dtype=torch.float32, device="cuda").normal_(0, 2, generator=g).to(torch.bfloat16)
    sw = torch.empty_like(gate)
    assert ref.ref_swiglu(gate.data_ptr(), up.data_ptr(), sw.data_ptr(), 4096, stream) == 0
    data["swiglu_gate"], data["swiglu_up"], data["swiglu_out"] = u16(gate), u16(up), u16(sw)
    mixed = torch.empty((3 * 8, 2560), dtype=torch.float32, device="cuda").normal_(0, 0.05, generator=g).to(torch.bfloat16)
    rw = torch.rand((3, 8), dtype=torch.float32, device="cuda", generator=g)
    comb = torch.empty((3, 2560), dtype=torch.bfloat16, device="cuda")
    assert ref.ref_expert_combine_rows(mixed.data_ptr(), rw.data_ptr(), comb.data_ptr(), 3, 8, 2560, stream) == 0
    data["combine_rows"], data["combine_weights"], data["combine_out"] = u16(mixed), rw.cpu().numpy(), u16(comb)

    # whole block on the synthetic layer (seed 1234, layer 0)
    layer = synth.make_layer(SEED, LAYER, keep_raw=True)
    raw = layer.raw
    digest = hashlib.sha256()
    for t in (raw.packed[:9], raw.scales_linear[:9], raw.packed[-3:], raw.alpha):
        digest.update(t.cpu().numpy().tobytes())
    data["layer_digest"] = np.frombuffer(digest.digest(), dtype=np.uint8)
    alphas = raw.alpha.cpu().numpy()
    for rows in (1, 4):
        x = synth.make_activations(SEED, 200 + rows, rows)
        out = torch.empty_like(x)
        ids = torch.empty((rows, 8), dtype=torch.int32, device="cuda")
        w = torch.empty((rows, 8), dtype=torch.float32, device="cuda")
        code = ref.ref_moe_forward_rows(x.data_ptr(), layer.router_weight.data_ptr(), layer.bias.data_ptr(),
                                        raw.packed.data_ptr(), raw.scales_linear.data_ptr(), alphas, raw.packed.shape[1],
                                        raw.scales_linear.shape[1], out.data_ptr(), rows, 2560, 1024, 256, 2.5, None,
                                        ids.data_ptr(), w.data_ptr(), None, stream)
        assert code == 0
        data[f"block{rows}_x"], data[f"block{rows}_out"] = u16(x), u16(out)
        data[f"block{rows}_ids"], data[f"block{rows}_weights"] = ids.cpu().numpy(), w.cpu().numpy()
    np.savez_compressed(out_path, **data)
    print("wrote", out_path, {k: v.shape for k, v in data.items()})


if __name__ == "__main__":
    main()
