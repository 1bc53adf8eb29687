"""CPU tests of the host-side pieces around the kernels: the constant container and the kernel database."""
import json
import os

import numpy as np
import pytest

from nnfusion_b200 import _lib as L
from nnfusion_b200 import constants, kernel_db, synth


def test_constant_container_roundtrip(tmp_path):
    rng = np.random.Generator(np.random.PCG64(1))
    w4 = synth.make_weights(rng, 48, 384, 4, 128)
    w8 = synth.make_weights(rng, 16, 256, 8, 256, np.float32, (0.001, 0.01), (120, 136))
    d = str(tmp_path)
    paths = constants.save_linear(d, "layers.0.mlp.up", w4)
    constants.save_linear(d, "lm_head", w8)
    # raw dumps named after the tensors, as Constant::emit_function_body writes them
    assert os.path.basename(paths["wq"]) == "layers.0.mlp.up.wq.bin"
    assert os.path.getsize(paths["wq"]) == 48 * 384 // 2
    info = json.load(open(os.path.join(d, "para_info.json")))
    e = info["weight"]["layers.0.mlp.up.wq"]
    assert e["shape"] == [48, 192] and e["id"].startswith("((uint8*)")      # packed uint4 travels as uint8
    assert info["weight"]["layers.0.mlp.up.scale"]["id"].startswith("((half*)")
    assert info["weight"]["lm_head.scale"]["id"].startswith("((float*)")
    assert info["quant"]["lm_head"] == {"N": 16, "K": 256, "w_bits": 8, "group_size": 256}
    for name, w in (("layers.0.mlp.up", w4), ("lm_head", w8)):
        r = constants.load_linear_host(d, name)
        assert (r.N, r.K, r.bits, r.group) == (w.N, w.K, w.bits, w.group)
        np.testing.assert_array_equal(r.q, w.q)
        np.testing.assert_array_equal(r.zp, w.zp)
        np.testing.assert_array_equal(np.asarray(r.scale), w.scale)
        np.testing.assert_array_equal(np.asarray(r.wq), w.wq)               # byte-identical: no re-layout


def test_constant_container_rejects_damage(tmp_path):
    rng = np.random.Generator(np.random.PCG64(2))
    d = str(tmp_path)
    paths = constants.save_linear(d, "q", synth.make_weights(rng, 16, 128, 4, 128))
    with pytest.raises(KeyError):
        constants.load_linear_host(d, "missing")
    with open(paths["scale"], "ab") as f:
        f.write(b"\0\0")
    with pytest.raises(ValueError, match="bytes on disk"):
        constants.load_linear_host(d, "q")


def test_odd_group_count_zero_points(tmp_path):
    rng = np.random.Generator(np.random.PCG64(3))
    w = synth.make_weights(rng, 8, 384, 4, 128)       # 3 groups: the last zero-point byte is half used
    constants.save_linear(str(tmp_path), "w", w)
    r = constants.load_linear_host(str(tmp_path), "w")
    assert r.zpq.shape == (8, 2)
    np.testing.assert_array_equal(r.zp, w.zp)


def test_identifier_follows_the_reference_recipe():
    ident = kernel_db.identifier(1, 11008, 4096, 4, 128, L.F16, L.F16, L.F16)
    # op type, then shapes of inputs ; output joined with , and ; then the dtypes
    # (element_type::c_type_string(): "half", "float", and "uint8_t" for u8 -- src/nnfusion/common/type/element_type.cpp:28-35;
    # concatenated by KernelContext::generate_identifier, src/nnfusion/core/kernels/kernel_emitter.cpp:415-455)
    assert ident == "DequantDot1,4096;11008,2048;11008,32;11008,16;1,11008halfuint8_thalfuint8_thalf"
    assert kernel_db.identifier(16, 4096, 4096, 8, 4096, L.F32, L.F32, L.F32).endswith("floatuint8_tfloatuint8_tfloat")
    assert ident != kernel_db.identifier(2, 11008, 4096, 4, 128, L.F16, L.F16, L.F16)


def test_kernel_db_schema_and_fetch(tmp_path):
    db = kernel_db.KernelCacheManager(str(tmp_path / "kernel_cache.db"))
    cols = [r[1] for r in db.db.execute("PRAGMA table_info(KernelCache)")]
    assert cols == ["Key", "Identifier", "OpType", "Attributes", "Source", "DeviceType", "Function", "Tags", "Miscs"]
    ident = kernel_db.identifier(8, 4096, 4096, 4, 128, L.F16, L.F16, L.F16)
    times = {(L.KERNEL_GEMV, 0): 9.0, (L.KERNEL_GEMV, 2): 7.5, (L.KERNEL_GEMM, 0): 21.0}

    def measure(fn):
        return times.get((fn["kernel"], fn["split_k"]))      # None: the library refuses the combination

    best = kernel_db.tune(db, ident, kernel_db.default_candidates(8), measure, "B200")
    assert best.function == {"kernel": L.KERNEL_GEMV, "split_k": 2}
    assert len(db.fetch_all(ident)) == 3                      # refused candidates are not stored
    assert db.fetch_with_tags(ident, kernel_db.DEVICE_TYPE, {"other"}, "B200") is None
    assert db.fetch_with_tags("DequantDot-unknown", kernel_db.DEVICE_TYPE, {"fast"}, "B200") is None
    # an entry without a time for this device loses against one that has it
    e = kernel_db.KernelEntry(identifier=ident, function={"kernel": L.KERNEL_GEMM, "split_k": 0}, tags={"fast"},
                              miscs={"external_profile": {"time": {"H100": 1.0}}})
    assert db.insert_kernel_entry(e, overwrite=True)
    assert db.fetch_with_tags(ident, kernel_db.DEVICE_TYPE, {"fast"}, "B200").function["split_k"] == 2
    assert not db.insert_kernel_entry(e)                      # same key, no overwrite
    db.close()
    # persistent: a new manager on the same file sees the entries
    assert len(kernel_db.KernelCacheManager(str(tmp_path / "kernel_cache.db")).fetch_all(ident)) == 3


def test_front_door_module_on_cpu_is_plain_pytorch():
    import torch
    from nnfusion_b200.jit import QuantLinear
    from oracle import oracle as orc

    rng = np.random.Generator(np.random.PCG64(5))
    w = synth.make_weights(rng, 24, 256, 4, 128)
    m = QuantLinear.from_host(w)
    np.testing.assert_allclose(m.dequantized().numpy(), orc.np_dequant(w.q, w.scale, w.zp, 128), rtol=0, atol=0)
    assert set(m.state_dict()) == {"wq", "scale", "zp"}
    with pytest.raises(RuntimeError, match="CUDA"):
        m(torch.zeros(1, 256, dtype=torch.float16))           # no CPU fallback
