"""CPU-only checks: format helpers, sizing contracts, plan builder shape, and that the C-ABI library loads
and exports every symbol include/swlm.h declares (no compute calls without a GPU)."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_pack_unpack_roundtrip(pkg):
    rng = np.random.default_rng(0)
    q = rng.integers(0, 16, size=(5, 192), dtype=np.uint8)
    w = pkg.pack_mlx_q4(q)
    assert w.shape == (5, 24) and w.dtype == np.uint32
    assert np.array_equal(pkg.formats.unpack_mlx_q4(w, 192), q)
    # element j of a row is nibble j%8 of word j/8, i.e. byte j/2, low nibble for even j
    raw = w.view(np.uint8).reshape(5, 96)
    assert np.array_equal(raw & 0xF, q[:, 0::2]) and np.array_equal(raw >> 4, q[:, 1::2])


def test_staf_block_geometry(pkg):
    fmt = pkg.AffineQ4Group64Format
    # Tests/MetalCompilerTests/Core/SupportedQuantizationsContractTests.swift:95-113 (block geometry)
    assert (fmt.bits, fmt.group_size, fmt.weights_per_block, fmt.bytes_per_block) == (4, 64, 64, 36)
    assert fmt.bytes_per_block == 4 + fmt.weights_per_block * fmt.bits // 8
    assert fmt.bytes_per_weight() == 0.5625


def test_kv_cache_sizing_contract(pkg):
    # Tests/MetalCompilerTests/Core/KVCacheSizingContractTests.swift:32-53, 129-185
    spec = pkg.KVCacheSpecification(layer_count=32, kv_head_count=8, head_dimension=128, maximum_sequence_length=4224)
    assert spec.bytes_per_head_slot() == 256
    assert spec.bytes_per_token_slot() == 8 * 256
    assert spec.bytes_per_layer() % spec.bytes_per_head_slot() == 0
    assert spec.total_bytes() == 553_648_128
    small = pkg.KVCacheSpecification(layer_count=6, kv_head_count=8, head_dimension=64, maximum_sequence_length=16)
    assert small.bytes_per_head_slot() == 256  # 128 bytes of data aligned up to the 256-byte dense slot
    assert small.sequence_major_offset(1, 2, 3) == 1 * 8 * 16 * 256 + 2 * 16 * 256 + 3 * 256


def test_kv_cache_sizing_of_block_and_rotated_schemes(pkg):
    # Tests/MetalCompilerTests/Core/KVCacheSizingContractTests.swift:32-80, 100-125 (rotated schemes size like their base);
    # Tests/MetalCompilerTests/Models/RotorQuant/RotorQuantCorrectnessTests.swift:52-67, 163-202
    def spec(scheme, hd=128, layers=16, seq=4096):
        return pkg.KVCacheSpecification(layer_count=layers, kv_head_count=8, head_dimension=hd, maximum_sequence_length=seq, scheme=scheme)
    assert spec(0x00).bytes_per_head_slot() == 256 and spec(0x01, hd=192).bytes_per_head_slot() == 512 and spec(0x02).bytes_per_head_slot() == 512
    assert spec(0x10).bytes_per_head_slot() == 192     # 4 blocks x 36 = 144 -> 64-byte slots
    assert spec(0x11).bytes_per_head_slot() == 192     # 2 x 68 = 136
    assert spec(0x40).bytes_per_head_slot() == 128     # 2 x 36 = 72
    assert spec(0x42).bytes_per_head_slot() == 128     # 1 x 68
    assert spec(0x70).bytes_per_head_slot() == spec(0x10).bytes_per_head_slot() and spec(0x71).bytes_per_head_slot() == spec(0x40).bytes_per_head_slot()
    assert spec(0x70).uses_rotor_quant and spec(0x71).uses_rotor_quant and not spec(0x10).uses_rotor_quant and not spec(0x01).uses_rotor_quant
    assert [spec(0x70, hd=h).num_rotor_groups() for h in (3, 4, 6, 64, 128, 1)] == [1, 2, 2, 22, 43, 1]
    r = spec(0x70)
    assert r.rotor_parameters_bytes_per_layer() == 8 * 43 * 4 * 2 and r.total_rotor_parameters_size() == 8 * 43 * 4 * 2 * 16
    assert r.qjl_matrix_size(16) == 128 * 16 * 2
    assert r.qjl_residual_bytes_per_layer(16) == 4096 * 8 * 16 * 2 and r.total_qjl_residual_size(16) == 4096 * 8 * 16 * 2 * 16
    assert r.qjl_matrix_size(0) == 0 and r.qjl_residual_bytes_per_layer(0) == 0 and r.total_qjl_residual_size(0) == 0
    # the C header's helpers agree on the unpadded rows this build stores (144 / 72 bytes for head_dim 128)
    desc = pkg.ModelConfig(family="llama", hidden=256, intermediate=512, layers=2, heads=4, kv_heads=2, head_dim=128, vocab=512,
                           max_seq=64, kv_scheme=0x71, kv_qjl_dim=16).buffers_desc()
    assert desc.kv_scheme == 0x71 and desc.kv_qjl_dim == 16


def test_llama_plan_shape(pkg):
    cfg = pkg.llama3_8b_config()
    b = pkg.DispatchPlanBuilder(cfg)
    steps = b.decode_steps()
    kinds = [s.kind for s in steps]
    P = pkg.plan
    # embed + 32 x (norm, q, k, v, attn, o, norm, gate, up, swiglu, down) + final norm + lm_head + argmax
    assert len(steps) == 1 + 32 * 11 + 3
    assert kinds[0] == P.STEP_EMBED and kinds[1] == P.STEP_COPY_RMSNORM
    assert kinds.count(P.STEP_QGEMV) == 32 * 7 + 1
    assert kinds.count(P.STEP_RESADD_COPY_RMSNORM) == 63 and kinds[-3:] == [P.STEP_RESADD_RMSNORM, P.STEP_QGEMV, P.STEP_ARGMAX]
    assert cfg.slot_dim == 16384
    assert cfg.q4_weight_elems() == 7_504_658_432
    assert int(cfg.q4_weight_elems() * 0.5625) == 4_221_370_368
    # the step count does not depend on the token count (Tests/MetalCompilerTests/Core/PrefillTests.swift:49-71)
    assert len(pkg.DispatchPlanBuilder(pkg.llama3_8b_config(max_seq=128)).decode_steps()) == len(steps)
    names = {t[0] for t in b.tensors()}
    for s in steps:
        if s.weight:
            assert s.weight.decode() in names


def test_lfm2_plan_shape(pkg):
    cfg = pkg.lfm2_like_config()
    b = pkg.DispatchPlanBuilder(cfg)
    steps = b.decode_steps()
    P = pkg.plan
    kinds = [s.kind for s in steps]
    assert cfg.kv_layer_count == 6 and cfg.conv_layer_count == 10
    assert kinds.count(P.STEP_CONV_STATE_UPDATE) == 10 and kinds.count(P.STEP_ATTN_DECODE) == 6
    assert kinds.count(P.STEP_QK_NORM) == 6
    conv_layers = [s.layer for s in steps if s.kind == P.STEP_CONV_STATE_UPDATE]
    assert conv_layers == list(range(10))
    assert cfg.q4_weight_elems() == 16 * 50_331_648 + 10 * 16_777_216 + 6 * 10_485_760 + 134_217_728


def test_deltanet_plan_shape_windows_and_cache_scheme(pkg):
    """The hybrid recurrent recipe: per recurrent layer four projections of one input, the recurrence step with its
    four buffers and four tensors, the out projection; every name the steps use is in the tensor inventory with the
    right kind; sliding windows and the cache scheme travel through the plan and the buffer description."""
    import dataclasses
    P = pkg.plan
    cfg = pkg.ModelConfig("deltanet", hidden=256, intermediate=512, layers=6, heads=4, kv_heads=2, head_dim=64, vocab=1024,
                          attention_layers=[2, 5], max_seq=64, ssm_heads=8, ssm_groups=4, ssm_key_dim=32, ssm_value_dim=64,
                          ssm_conv_kernel=4, sliding_window=16, sliding_window_layers=[5], kv_scheme=0x11)
    b = pkg.DispatchPlanBuilder(cfg)
    steps = b.decode_steps()
    kinds = [s.kind for s in steps]
    assert cfg.ssm_layer_count == 4 and cfg.kv_layer_count == 2 and cfg.conv_layer_count == 0
    assert cfg.ssm_conv_dim == 2 * 4 * 32 + 8 * 64 and cfg.slot_dim >= cfg.ssm_conv_dim
    assert kinds.count(P.STEP_SSM_RECURRENCE) == 4 and kinds.count(P.STEP_ATTN_DECODE) == 2
    assert kinds.count(P.STEP_QGEMV) == 4 * 5 + 2 * 4 + 6 * 3 + 1
    rec = [s for s in steps if s.kind == P.STEP_SSM_RECURRENCE]
    assert [s.layer for s in rec] == [0, 1, 2, 3]
    r0 = rec[0]
    assert (r0.in_buf, r0.in2_buf, r0.in3_buf, r0.in4_buf, r0.out_buf) == (P.BUF_S1, P.BUF_S2, P.BUF_S3, P.BUF_S4, P.BUF_S0)
    assert (r0.heads, r0.groups, r0.key_dim, r0.value_dim, r0.conv_kernel) == (8, 4, 32, 64, 4)
    assert r0.weight.decode().endswith("linear_attn.conv1d.weight") and r0.weight4.decode().endswith("linear_attn.A_log")
    kinds_by_name = {t[0]: t[1] for t in b.tensors()}
    assert kinds_by_name[r0.weight2.decode()] == "f32" and kinds_by_name[r0.weight4.decode()] == "f32"
    assert kinds_by_name[r0.weight.decode()] == "conv" and kinds_by_name[r0.weight3.decode()] == "dense"
    for s in steps:
        for w in (s.weight, s.weight2, s.weight3, s.weight4):
            if w:
                assert w.decode() in kinds_by_name
    att = [s for s in steps if s.kind == P.STEP_ATTN_DECODE]
    assert [s.window_left for s in att] == [0, 16]                 # only model layer 5 is windowed
    d = cfg.buffers_desc()
    assert (d.ssm_layers, d.ssm_heads, d.ssm_groups, d.ssm_key_dim, d.ssm_value_dim, d.ssm_conv_kernel, d.kv_scheme) == (4, 8, 4, 32, 64, 4, 0x11)
    plain = dataclasses.replace(cfg, family="llama", attention_layers=[]).buffers_desc()
    assert plain.ssm_layers == 0 and plain.ssm_heads == 0
    w = pkg.synth_model_weights(b, seed=1)
    assert w[r0.weight2.decode()].dtype == np.float32 and w[r0.weight3.decode()].dtype == np.uint16
    assert abs(float(w[r0.weight4.decode()].min())) <= 1.0


def test_synth_distributions(pkg):
    w, s, b = pkg.synth_q4(64, 4096, seed=0)
    q = pkg.formats.unpack_mlx_q4(w, 4096)
    assert q.min() == 0 and q.max() == 15 and abs(q.mean() - 7.5) < 0.05
    sf, bf = pkg.bf16_to_f32(s), pkg.bf16_to_f32(b)
    assert 0.00498 <= sf.min() and sf.max() <= 0.0201
    assert abs(bf.std() - 0.01) < 0.001
    w2, _, _ = pkg.synth_q4(64, 4096, seed=0)
    assert np.array_equal(w, w2)


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "swlm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(swlm_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    syms = _declared_symbols()
    assert len(syms) >= 35
    lib = pkg.load_library()  # raises if the .so is missing: there is no fallback
    for s in syms:
        assert hasattr(lib.dll, s), f"{s} declared in include/swlm.h but not exported"
        assert s in pkg.lib.SIGNATURES, f"{s} has no ctypes signature"
    assert lib.swlm_version().startswith(b"swlm-cuda")


def test_no_device_means_error_not_fallback(pkg):
    lib = pkg.load_library()
    if lib.swlm_device_count() > 0:
        pytest.skip("a CUDA device is present")
    h = ctypes.c_void_p()
    rc = lib.swlm_ctx_create(0, 0, 1, ctypes.byref(h))
    assert rc != 0 and not h.value
    assert b"no CUDA device" in lib.swlm_last_error()
    with pytest.raises(pkg.SwlmError):
        pkg.WeightStore(0)


def test_bad_arguments_are_rejected(pkg):
    lib = pkg.load_library()
    h = ctypes.c_void_p()
    assert lib.swlm_ctx_create(0, 3, 2, ctypes.byref(h)) == -1  # rank outside the group
    assert lib.swlm_position(None) == -1
    assert lib.swlm_plan_launch_count(None) == 0


def test_kv_cache_schemes_the_library_accepts(pkg):
    """KVCacheKernelSupportContractTests 'isSupportedForKVCache matches the pinned supported set'
    (Tests/MetalCompilerTests/Core/KVCacheKernelSupportContractTests.swift:20-50): the reference's attention kernels read
    and write fp16 / bf16 / fp32, q4 g64 / g128 / g128zero, q8 g32 / g64 / g128 and the two rotated schemes, and nothing
    else. This library offers that set without the dense fp16 and fp32 caches (its activations are bf16), 0 standing
    for "unset" = bf16; the sizable-but-unsupported schemes of the reference are refused here as well."""
    lib = pkg.load_library()
    reference_supported = {0x00, 0x01, 0x02, 0x40, 0x41, 0x42, 0x10, 0x11, 0x12, 0x71, 0x70}
    here = {s for s in range(0x100) if lib.swlm_kv_scheme_supported(s)}
    assert here == (reference_supported - {0x02}) and lib.swlm_kv_scheme_supported(0x00)    # (0 accepted as "unset", not as fp16)
    for scheme in here - {0x00, 0x01}:
        spec = pkg.KVCacheSpecification(layer_count=1, kv_head_count=1, head_dimension=128, maximum_sequence_length=1, scheme=scheme)
        assert spec.bytes_per_head_slot() % 64 == 0 and spec.bytes_per_head_slot() < 256     # every accepted block scheme is sizable


def test_tensor_parallel_head_split_is_checked(pkg):
    """Heads and KV heads must divide by the number of ranks, and every rank must keep whole GQA groups; anything else
    would silently compute with truncated head counts, so it is refused (host-only entry point; swlm_plan_build applies
    the same check to every attention and QK-norm step)."""
    lib = pkg.load_library()
    ok, unsupported = 0, -4
    assert lib.swlm_tp_check_heads(32, 8, 1) == ok
    assert lib.swlm_tp_check_heads(32, 8, 2) == ok
    assert lib.swlm_tp_check_heads(32, 8, 8) == ok       # one KV head per rank
    assert lib.swlm_tp_check_heads(8, 4, 8) == unsupported   # half a KV head per rank
    assert lib.swlm_tp_check_heads(12, 4, 8) == unsupported  # query heads do not divide
    assert lib.swlm_tp_check_heads(12, 6, 4) == unsupported
    assert lib.swlm_tp_check_heads(24, 8, 4) == ok
    assert b"GQA" in lib.swlm_last_error() or True
    assert lib.swlm_tp_check_heads(0, 8, 2) == -1
