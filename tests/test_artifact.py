"""The engine's NVFP4 weight container ("P92FP41", include/p92/nvfp4_artifact.h) and the loader that turns a layer
of it into an expert bank (src/resident.cpp:75-162, src/model.cpp:772-805).  No real checkpoint exists in this
build, so every test writes a synthetic container itself, in the layout the reference's packer writes
(cuda/nvfp4_pack.cu:264-305): the reader is tested on CPU, the loader on a GPU against the CPU oracle fed with the
same bytes."""
import os
import struct

import numpy as np
import pytest

from conftest import from_u16, u16

MAGIC = b"P92FP41\0"


def write_container(directory, tensors, swizzled=None, order=None, align=4096, header_patch=None, record_patch=None):
    """tensors: {name: (packed uint8 [rows, cols/2], scales uint8 [rows, cols/16], weight_scale_2)}."""
    names = order or sorted(tensors, key=lambda n: n.encode())
    records, weights, scales, tiled = [], bytearray(), bytearray(), bytearray()
    for name in names:
        packed, sc, alpha = tensors[name]
        for blob in (weights, scales, tiled):
            blob.extend(b"\0" * (-len(blob) % align))
        rows, cols = packed.shape[0], packed.shape[1] * 2
        rec = [name.encode().ljust(96, b"\0"), rows, cols, len(weights), len(scales), float(alpha), 0]
        if record_patch and name in record_patch:
            rec = record_patch[name](rec)
        records.append(struct.pack("<96sIIQQfI", *rec))
        weights.extend(packed.tobytes())
        scales.extend(sc.tobytes())
        tiled.extend((swizzled[name] if swizzled else sc).tobytes())
    header = [MAGIC, 1, 128, len(records), 0, len(weights), len(scales), 12345]
    if header_patch:
        header = header_patch(header)
    os.makedirs(directory, exist_ok=True)
    with open(os.path.join(directory, "manifest.bin"), "wb") as f:
        f.write(struct.pack("<8sIIIIQQQ", *header) + b"".join(records))
    open(os.path.join(directory, "weights.nvfp4"), "wb").write(bytes(weights))
    open(os.path.join(directory, "scales.e4m3"), "wb").write(bytes(scales))
    if swizzled is not None:
        open(os.path.join(directory, "scales.swizzled.e4m3"), "wb").write(bytes(tiled))


def tiny_tensors(rng, names, rows=128, cols=64):
    return {n: (rng.integers(0, 256, (rows, cols // 2), dtype=np.uint8), rng.integers(0, 120, (rows, cols // 16), dtype=np.uint8),
                0.001 * (i + 1)) for i, n in enumerate(names)}


# ------------------------------------------------------------------ reader (no GPU)

def test_reader_finds_records_by_name_and_returns_their_bytes(pkg, tmp_path):
    pkg.load_library()
    rng = np.random.default_rng(1)
    names = ["model.layers.2.mlp.experts.10.up_proj.weight", "lm_head.weight", "model.layers.2.mlp.experts.9.up_proj.weight",
             "model.layers.2.mlp.shared_experts.down_proj.weight", "a"]
    tensors = tiny_tensors(rng, names)
    write_container(str(tmp_path), tensors)
    art = pkg.Nvfp4Artifact(str(tmp_path))
    assert art.tensor_count == 5 and not art.has_swizzled_scales
    listed = [art.at(i).name.decode() for i in range(5)]
    assert listed == sorted(names, key=lambda n: n.encode())            # byte order, as the reference's binary search needs
    for name, (packed, scales, alpha) in tensors.items():
        rec = art.find(name)
        assert (rec.rows, rec.columns) == (128, 64) and rec.weight_offset % 4096 == 0
        assert rec.weight_scale_2 == np.float32(alpha)
        assert art.weight_bytes(rec) == packed.tobytes() and art.scale_bytes(rec) == scales.tobytes()
    with pytest.raises(pkg.P92Error) as err:
        art.find("model.layers.2.mlp.experts.11.up_proj.weight")
    assert "missing NVFP4 tensor" in str(err.value)
    with pytest.raises(pkg.P92Error):
        art.at(5)
    art.close()
    # with the optional pre-tiled scale file
    write_container(str(tmp_path / "tiled"), tensors, swizzled={n: t[1] for n, t in tensors.items()})
    art = pkg.Nvfp4Artifact(str(tmp_path / "tiled"))
    assert art.has_swizzled_scales
    art.close()


@pytest.mark.parametrize("case", ["magic", "version", "record_bytes", "count", "weight_size", "order", "rows", "columns", "alpha",
                                  "extent", "missing_file", "tiled_size"])
def test_reader_rejects_what_the_reference_reader_rejects(pkg, tmp_path, case):
    """src/nvfp4_artifact.cpp:76-106 and src/resident.cpp:104-107, one violation each."""
    pkg.load_library()
    rng = np.random.default_rng(2)
    names = ["b", "c", "d"]
    tensors = tiny_tensors(rng, names)
    kw, message = {}, None
    if case == "magic":
        kw["header_patch"], message = (lambda h: [b"P92FP40\0"] + h[1:]), "contract mismatch"
    elif case == "version":
        kw["header_patch"], message = (lambda h: h[:1] + [2] + h[2:]), "contract mismatch"
    elif case == "record_bytes":
        kw["header_patch"], message = (lambda h: h[:2] + [64] + h[3:]), "contract mismatch"
    elif case == "count":
        kw["header_patch"], message = (lambda h: h[:3] + [4] + h[4:]), "contract mismatch"
    elif case == "weight_size":
        kw["header_patch"], message = (lambda h: h[:5] + [h[5] + 16] + h[6:]), "file-size mismatch"
    elif case == "order":
        kw["order"], message = ["c", "b", "d"], "invalid NVFP4 record"
    elif case == "rows":
        kw["record_patch"], message = {"c": lambda r: r[:1] + [64] + r[2:]}, "invalid NVFP4 record"
    elif case == "columns":
        kw["record_patch"], message = {"c": lambda r: r[:2] + [72] + r[3:]}, "invalid NVFP4 record"
    elif case == "alpha":
        kw["record_patch"], message = {"c": lambda r: r[:5] + [0.0] + r[6:]}, "invalid NVFP4 record"
    elif case == "extent":
        kw["record_patch"], message = {"d": lambda r: r[:3] + [r[3] + 4096] + r[4:]}, "outside artifact"
    write_container(str(tmp_path), tensors, **kw)
    if case == "missing_file":
        os.remove(str(tmp_path / "scales.e4m3"))
        message = "cannot open"
    if case == "tiled_size":
        open(str(tmp_path / "scales.swizzled.e4m3"), "wb").write(b"\0" * 64)
        message = "pre-swizzled scale file size mismatch"
    with pytest.raises(pkg.P92Error) as err:
        pkg.Nvfp4Artifact(str(tmp_path))
    assert message in str(err.value)
    assert err.value.code == (301 if case == "missing_file" else 1)


# ------------------------------------------------------------------ loader (GPU)

HIDDEN, INTER = 256, 512          # a small expert shape the tile stream supports: the container logic does not depend on it


def _quantised(orc, rng, rows, cols):
    w = orc.f32_to_bf16((rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(0.05)))
    packed, scales, alpha = orc.nvfp4_pack_weight(w)
    return packed, scales, alpha


def _moe_layer_tensors(orc, seed, layer):
    rng = np.random.default_rng(seed)
    tensors, order = {}, []
    prefixes = [f"model.layers.{layer}.mlp.experts.{e}" for e in range(256)] + [f"model.layers.{layer}.mlp.shared_experts"]
    for prefix in prefixes:
        for kind, (rows, cols) in (("gate_proj", (INTER, HIDDEN)), ("up_proj", (INTER, HIDDEN)), ("down_proj", (HIDDEN, INTER))):
            name = f"{prefix}.{kind}.weight"
            tensors[name] = _quantised(orc, rng, rows, cols)
            order.append(name)
    return tensors, order


@pytest.mark.gpu
@pytest.mark.parametrize("tiled", [False, True])
def test_bank_loaded_from_a_container_computes_what_the_oracle_computes_from_the_same_bytes(cuda, pkg, orc, tmp_path, tiled):
    torch = cuda
    pkg.load_library()
    layer = 2
    tensors, order = _moe_layer_tensors(orc, 5, layer)
    # an unrelated tensor of another shape in between: the loader must pick by name, not by position
    tensors["model.layers.2.self_attn.o_proj.weight"] = tiny_tensors(np.random.default_rng(0), ["x"], 256, 128)["x"]
    swz = {n: orc.swizzle_scales(t[1]).reshape(t[1].shape) for n, t in tensors.items()} if tiled else None
    write_container(str(tmp_path), tensors, swizzled=swz)
    art = pkg.Nvfp4Artifact(str(tmp_path))
    assert art.has_swizzled_scales == tiled
    bank = art.load_bank(layer)
    art.close()                                                    # the bank keeps nothing of the mapping
    rng = np.random.default_rng(6)
    router = orc.f32_to_bf16((rng.standard_normal((256, HIDDEN), dtype=np.float32) * np.float32(0.08)))
    bias = (rng.standard_normal(256) * 0.01).astype(np.float32)
    packed = np.stack([tensors[n][0].reshape(-1) for n in order])
    scales = np.stack([tensors[n][1].reshape(-1) for n in order])
    alphas = np.array([tensors[n][2] for n in order], np.float32)
    for rows in (6, 40):
        x = orc.f32_to_bf16(rng.standard_normal((rows, HIDDEN), dtype=np.float32))
        plan = pkg.MoePlan(max_rows=rows, hidden=HIDDEN, intermediate=INTER)
        out = torch.full((rows, HIDDEN), float("nan"), dtype=torch.bfloat16, device="cuda")
        block = pkg.MoeBlock(bank, from_u16(router), torch.from_numpy(bias).cuda(), plan)
        block.run_moe_rows(from_u16(x), out, rows)
        torch.cuda.synchronize()
        assert plan.status() == 0
        want, extra = orc.moe_forward(x, router, bias, packed, scales, alphas, HIDDEN, INTER, want_intermediates=True)
        _, _, margin = orc.router_top8(extra["logits"], bias)
        safe = margin > 2e-6
        ids = plan.views(rows)["expert_ids"].cpu().numpy()
        assert np.array_equal(ids[safe], extra["expert_ids"][safe])
        got, exp = orc.bf16_to_f32(u16(out))[safe], orc.bf16_to_f32(want)[safe]
        assert np.isfinite(got).all()
        rel = float(np.linalg.norm(got - exp) / np.linalg.norm(exp))
        assert rel <= 1e-2 and float(np.abs(got - exp).max()) <= 2e-2, (rows, rel)
        plan.close()
    # an expert-parallel shard of the same container: experts 64..127
    art = pkg.Nvfp4Artifact(str(tmp_path))
    shard = art.load_bank(layer, first_expert=64, local_experts=64)
    assert shard.nbytes < bank.nbytes
    with pytest.raises(pkg.P92Error) as err:
        art.load_bank(7)                                           # no such layer in the container
    assert "missing NVFP4 tensor" in str(err.value)
    art.close()
    shard.close()
    bank.close()


@pytest.mark.gpu
def test_dense_bank_loaded_from_a_container(cuda, pkg, orc, tmp_path):
    torch = cuda
    pkg.load_library()
    rng = np.random.default_rng(8)
    inter = 1024
    names = [f"model.layers.0.mlp.{k}.weight" for k in ("gate_proj", "up_proj", "down_proj")]
    shapes = [(inter, HIDDEN), (inter, HIDDEN), (HIDDEN, inter)]
    tensors = {n: _quantised(orc, rng, *s) for n, s in zip(names, shapes)}
    write_container(str(tmp_path), tensors)
    art = pkg.Nvfp4Artifact(str(tmp_path))
    bank = art.load_dense_bank(0)
    rows = 9
    x = orc.f32_to_bf16(rng.standard_normal((rows, HIDDEN), dtype=np.float32))
    plan = pkg.MoePlan(max_rows=rows, hidden=HIDDEN, intermediate=inter)
    out = torch.full((rows, HIDDEN), float("nan"), dtype=torch.bfloat16, device="cuda")
    pkg.run_dense_rows(plan, bank, from_u16(x), out, rows)
    torch.cuda.synchronize()
    assert plan.status() == 0
    packed = np.stack([tensors[n][0].reshape(-1) for n in names])
    scales = np.stack([tensors[n][1].reshape(-1) for n in names])
    alphas = np.array([tensors[n][2] for n in names], np.float32)
    want = orc.bf16_to_f32(orc.dense_forward(x, packed, scales, alphas, HIDDEN, inter))
    got = orc.bf16_to_f32(u16(out))
    rel = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    assert np.isfinite(got).all() and rel <= 1e-2 and float(np.abs(got - want).max()) <= 2e-2, rel
    plan.close()
    bank.close()
    art.close()
