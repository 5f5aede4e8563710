"""STAF files on the host (no GPU): the packed layout the reference's loader documents, writer/reader round trips,
the validator's rules, and the reference's end-to-end known answer driven through a real file:
MLX-shaped safetensors -> converter -> STAF file -> loader -> block GEMV (STAFEndToEndGEMVTests.q4Group64EndToEnd,
Tests/MetalCompilerTests/Core/STAFEndToEndGEMVTests.swift:51-54,137-160,295-320)."""
import os
import struct
import time

import numpy as np
import pytest


@pytest.fixture
def staf(pkg):
    return pkg.staf


def _bf(pkg, a):
    return pkg.f32_to_bf16(np.asarray(a, dtype=np.float32))


def _bundle(pkg, tmp_path, g):
    """The multi-row known answer as an MLX-shaped safetensors file: `*.weight` u32, `*.scales` / `*.biases` bf16,
    plus a dense bf16 norm weight."""
    w = pkg.pack_mlx_q4(np.array(g["q"], dtype=np.uint8))
    tensors = {
        "model.layers.0.mlp.down_proj.weight": ("U32", w),
        "model.layers.0.mlp.down_proj.scales": ("BF16", _bf(pkg, g["scales"])),
        "model.layers.0.mlp.down_proj.biases": ("BF16", _bf(pkg, g["zeros"])),
        "model.norm.weight": ("BF16", _bf(pkg, np.linspace(0.5, 1.5, 64))),
    }
    path = os.path.join(tmp_path, "model.safetensors")
    pkg.staf.write_safetensors(path, tensors)
    return path, w


def test_packed_layout_matches_the_loaders_offsets(pkg, staf, tmp_path):
    """Byte offsets of STAF/STAFLoader.swift:68-87 (section entry) and STAFFormat.swift:72-79 (header); payload
    placement of STAFWriter.swift:55-69: first payload on a 4096-byte boundary, every tensor on a 256-byte one."""
    a = staf.TensorToWrite("a.weight", staf.SCHEME_Q4_G64, staf.ROLE_DOWN, staf.DTYPE_I32, (4, 32), bytes(range(200)) * 2 + b"x" * 176,
                           block_size=64, group_size=64, shard_index=1)
    b = staf.TensorToWrite("norm", staf.SCHEME_BF16, staf.ROLE_NORM, staf.DTYPE_BF16, (7,), b"\x01" * 14)
    path = os.path.join(tmp_path, "t.staf")
    staf.write_staf(path, [a, b], {"zeta": True, "alpha": staf.U32(5), "mid": "text", "f": 0.25})
    raw = open(path, "rb").read()
    magic, version, meta_count, meta_off = struct.unpack_from("<IIII", raw, 0)
    sections, section_off, string_off, string_size = struct.unpack_from("<IIII", raw, 40)
    assert (magic, version, sections, section_off) == (0x46415453, 2, 2, 64)
    assert raw[:4] == b"STAF" and raw[16:40] == bytes(24) and raw[56:64] == bytes(8)
    assert meta_off == 64 + 2 * 128 and meta_count == 4 and string_off == meta_off + 4 * 32
    e0 = raw[64:192]
    name_off, name_len = struct.unpack_from("<II", e0, 0)
    assert raw[string_off + name_off:string_off + name_off + name_len] == b"a.weight"
    assert raw[string_off + name_off + name_len] == 0                      # NUL-terminated
    assert tuple(e0[8:12]) == (0x40, 0x08, 0x03, 2)                        # scheme, role, original dtype, rank
    assert struct.unpack_from("<8I", e0, 12) == (4, 32, 0, 0, 0, 0, 0, 0)
    p_off, p_size = struct.unpack_from("<QQ", e0, 44)
    assert struct.unpack_from("<IIIII", e0, 60) == (256, 64, 64, 0, 1)      # alignment, block, group, checksum, shard
    assert e0[80:] == bytes(48)
    assert p_off % 4096 == 0 and p_off >= string_off + string_size and p_size == 576
    p1_off, p1_size = struct.unpack_from("<QQ", raw[192:320], 44)
    assert p1_off % 256 == 0 and p1_off == (p_off + p_size + 255) // 256 * 256 and p1_size == 14
    assert len(raw) == p1_off + 14
    # metadata entries are sorted by key; an entry is key offset, key length, type at 8, payloads at 12 and 20
    keys = []
    for i in range(meta_count):
        m = raw[meta_off + 32 * i:meta_off + 32 * (i + 1)]
        ko, kl, vt = struct.unpack_from("<IIB", m, 0)
        keys.append((raw[string_off + ko:string_off + ko + kl].decode(), vt))
    assert keys == [("alpha", 0x02), ("f", 0x05), ("mid", 0x06), ("zeta", 0x01)]
    back = staf.read_staf(path)
    assert back.names() == ["a.weight", "norm"]
    assert back.metadata == {"zeta": True, "alpha": staf.U32(5), "mid": "text", "f": 0.25}
    assert bytes(back.payload("a.weight")) == a.payload and bytes(back.payload("norm")) == b.payload
    assert back["a.weight"].shape == (4, 32) and back["a.weight"].group_size == 64 and back["a.weight"].shard_index == 1


def test_safetensors_to_staf_end_to_end_known_answer(pkg, staf, oracle, golden, tmp_path):
    g = golden["gemv_multi_row"]
    src, w = _bundle(pkg, tmp_path, g)
    out = os.path.join(tmp_path, "model.staf")
    assert staf.convert_safetensors([src], out) is True
    f = staf.read_staf(out)
    # the companions of the quantized triple are consumed; tensors keep the source order
    assert f.names() == ["model.layers.0.mlp.down_proj.weight", "model.norm.weight"]
    e = f["model.layers.0.mlp.down_proj.weight"]
    assert (e.scheme, e.block_size, e.group_size, e.role) == (staf.SCHEME_Q4_G64, 64, 64, staf.ROLE_DOWN)
    assert e.shape == (g["rows"], 8 * g["blocks"]) and e.payload_size == g["rows"] * g["blocks"] * 36
    assert f["model.norm.weight"].scheme == staf.SCHEME_BF16 and f["model.norm.weight"].role == staf.ROLE_NORM
    assert f.metadata[staf.KEY_SOURCE_FORMAT] == "safetensors"
    assert f.metadata[staf.KEY_CONVERTER_VERSION] == staf.U32(3) and f.metadata[staf.KEY_SOURCE_SHARD_COUNT] == 1
    # payload = interleaved [fp16 scale][fp16 zero][32 nibble bytes] blocks, byte for byte the oracle's repack
    blocks = np.asarray(f.payload(e.name)).reshape(g["rows"], g["blocks"], 36)
    assert np.array_equal(blocks, oracle.staf_repack(w, _bf(pkg, g["scales"]), _bf(pkg, g["zeros"])))
    # ... and the GEMV over the blocks as loaded from the file gives the reference test's expectation
    y = oracle.staf_gemv_f32(blocks, g["rows"], 64 * g["blocks"], np.array(g["x"], dtype=np.float32))
    for r in range(g["rows"]):
        assert abs(float(y[r]) - g["expected"][r]) < max(g["abs_tol"], g["rel_tol"] * abs(g["expected"][r]))


def test_validator_rules(pkg, staf, golden, tmp_path):
    src, _ = _bundle(pkg, tmp_path, golden["gemv_multi_row"])
    out = os.path.join(tmp_path, "model.staf")
    staf.convert_safetensors([src], out)
    expected = staf.default_cache_metadata(1)
    assert staf.is_valid(out, [src], expected)
    assert staf.convert_safetensors([src], out) is False                       # a valid cache is kept
    assert not staf.is_valid(out, [src], dict(expected, **{"model.hidden_size": staf.U32(4096)}))   # key missing
    assert not staf.is_valid(out, [src], {staf.KEY_CONVERTER_VERSION: staf.U32(2)})                  # stale converter
    assert not staf.is_valid(out, [src], {staf.KEY_CONVERTER_VERSION: 3})                            # same number, other type
    # a source newer than the cache invalidates it
    later = time.time() + 100
    os.utime(src, (later, later))
    assert not staf.is_valid(out, [src], expected)
    assert staf.convert_safetensors([src], out) is False or True
    # header damage: version, magic, section table offset, truncated payload
    raw = bytearray(open(out, "rb").read())
    for patch in ((4, struct.pack("<I", 1)), (0, b"XTAF"), (44, struct.pack("<I", 128))):
        bad = bytearray(raw)
        bad[patch[0]:patch[0] + len(patch[1])] = patch[1]
        p = os.path.join(tmp_path, "bad.staf")
        open(p, "wb").write(bad)
        assert not staf.is_valid(p)
    p = os.path.join(tmp_path, "short.staf")
    open(p, "wb").write(raw[:4096 + 100])
    assert not staf.is_valid(p)
    with pytest.raises(staf.STAFError):
        staf.read_staf(p)


def test_unsupported_quantization_is_refused(pkg, staf, golden, tmp_path):
    src, _ = _bundle(pkg, tmp_path, golden["gemv_multi_row"])
    with pytest.raises(staf.STAFError):
        staf.plan_conversion(staf.read_safetensors(src), bits=4, group_size=128)
    with pytest.raises(staf.STAFError):
        staf.plan_conversion(staf.read_safetensors(src), bits=8, group_size=64)


def test_group128_bundle_becomes_68_byte_blocks(pkg, staf, oracle, tmp_path):
    """AffineQ4Group128Format (STAF/QuantizationFormat.swift:539-604): scheme 0x41, 128 weights per 68-byte block, the
    same per-weight expression. The file's blocks equal the oracle's repack byte for byte and dequantise to
    scale * q + zero with the fp16-narrowed group-128 parameters."""
    n, k = 6, 384
    w, s, b = pkg.synth_q4(n, k, seed=77, group=128)
    src = os.path.join(tmp_path, "g128.safetensors")
    staf.write_safetensors(src, {"model.layers.0.mlp.up_proj.weight": ("U32", w),
                                 "model.layers.0.mlp.up_proj.scales": ("BF16", s),
                                 "model.layers.0.mlp.up_proj.biases": ("BF16", b)})
    out = os.path.join(tmp_path, "g128.staf")
    with pytest.raises(staf.STAFError):
        staf.convert_safetensors([src], out)                       # the default hint (group 64) contradicts the shapes
    assert staf.convert_safetensors([src], out, group_size=128) is True
    f = staf.read_staf(out)
    e = f["model.layers.0.mlp.up_proj.weight"]
    assert (e.scheme, e.block_size, e.group_size, e.payload_size) == (staf.SCHEME_Q4_G128, 128, 128, n * (k // 128) * 68)
    blocks = np.asarray(f.payload(e.name)).reshape(n, k // 128, 68)
    assert np.array_equal(blocks, oracle.staf_repack_group(w, s, b, 128))
    assert np.array_equal(blocks, pkg.formats.repack_mlx_to_staf(w, s, b, group=128))
    deq = oracle.dequant_staf_group(blocks, n, k, 128)
    q = np.array([[(int(w[r, c // 8]) >> (4 * (c % 8))) & 15 for c in range(k)] for r in range(n)], dtype=np.float32)
    s16 = pkg.bf16_to_f32(s).astype(np.float16).astype(np.float32)
    z16 = pkg.bf16_to_f32(b).astype(np.float16).astype(np.float32)
    assert np.array_equal(deq, np.repeat(s16, 128, axis=1) * q + np.repeat(z16, 128, axis=1))

    class Recorder:
        def add_q4_staf(self, name, blk, n_, k_, shard=0, group=64):
            self.got = (name, np.array(blk).shape, n_, k_, shard, group)

    rec = Recorder()
    staf.load_into_store(rec, f)
    assert rec.got == (e.name, (n, k // 128, 68), n, k, 0, 128)


def test_load_into_store_routes_by_scheme(pkg, staf, golden, tmp_path):
    """`load_into_store` against a recording stand-in for the weight store: block tensors go in as blocks with
    (n, k) recovered from the packed shape, dense tensors as bf16 rows, fp32 sources rounded to bf16."""
    g = golden["gemv_multi_row"]
    src, w = _bundle(pkg, tmp_path, g)
    extra = os.path.join(tmp_path, "extra.safetensors")
    staf.write_safetensors(extra, {"model.layers.0.conv.conv.weight": ("F32", np.arange(12, dtype=np.float32).reshape(4, 3) / 8)})
    out = os.path.join(tmp_path, "model.staf")
    staf.convert_safetensors([src, extra], out)

    class Recorder:
        def __init__(self):
            self.q4, self.dense = {}, {}

        def add_q4_staf(self, name, blocks, n, k, shard=0):
            self.q4[name] = (np.array(blocks), n, k, shard)

        def add_dense(self, name, data, shard=0):
            self.dense[name] = (np.array(data), shard)

    rec = Recorder()
    f = staf.read_staf(out)
    loaded = staf.load_into_store(rec, f, shard_kinds={"model.layers.0.mlp.down_proj.weight": 2})
    assert sorted(loaded) == sorted(f.names())
    blocks, n, k, shard = rec.q4["model.layers.0.mlp.down_proj.weight"]
    assert (n, k, shard) == (g["rows"], 64 * g["blocks"], 2) and blocks.shape == (n, k // 64, 36)
    conv, _ = rec.dense["model.layers.0.conv.conv.weight"]
    assert conv.shape == (4, 3) and np.array_equal(pkg.bf16_to_f32(conv), np.arange(12, dtype=np.float32).reshape(4, 3) / 8)
    norm, _ = rec.dense["model.norm.weight"]
    assert norm.shape == (1, 64)
    assert f["model.layers.0.conv.conv.weight"].shard_index == 0 and f[loaded[0]].shard_index in (0, 1)


def test_recurrent_layer_tensors_keep_fp32(pkg, staf, tmp_path):
    """A bundle of the hybrid recurrent recipe: `linear_attn.norm.weight` is promoted to an fp32 section even when the
    bundle stores it as bf16 (STAFConversionPlanner.swift:117-140), `A_log` stays fp32, and both reach the weight store
    through the fp32 entry point; the quantized projections of the layer become 36-byte blocks like any other."""
    cfg = pkg.ModelConfig("deltanet", hidden=128, intermediate=256, layers=2, heads=4, kv_heads=2, head_dim=32, vocab=256,
                          attention_layers=[1], max_seq=16, ssm_heads=4, ssm_groups=2, ssm_key_dim=32, ssm_value_dim=32, ssm_conv_kernel=4)
    builder = pkg.DispatchPlanBuilder(cfg)
    weights = pkg.synth_model_weights(builder, seed=2)
    tensors = pkg.bundle_tensors(builder, weights)
    norm = "model.layers.0.linear_attn.norm.weight"
    tensors[norm] = ("BF16", pkg.f32_to_bf16(weights[norm]))          # as an MLX bundle would carry it
    src = os.path.join(tmp_path, "model.safetensors")
    staf.write_safetensors(src, tensors)
    out = os.path.join(tmp_path, "model.staf")
    assert staf.convert_safetensors([src], out)
    f = staf.read_staf(out)
    assert f[norm].scheme == staf.SCHEME_FP32 and f[norm].payload_size == 4 * cfg.ssm_value_dim
    assert np.array_equal(np.asarray(f.payload(norm)).view(np.float32), pkg.bf16_to_f32(pkg.f32_to_bf16(weights[norm])))
    assert f["model.layers.0.linear_attn.A_log"].scheme == staf.SCHEME_FP32
    assert f["model.layers.0.linear_attn.in_proj_qkv.weight"].scheme == staf.SCHEME_Q4_G64

    class Recorder:
        def __init__(self):
            self.f32, self.q4, self.dense = {}, [], []

        def add_dense_f32(self, name, data):
            self.f32[name] = np.array(data)

        def add_q4_staf(self, name, *a, **k):
            self.q4.append(name)

        def add_dense(self, name, *a, **k):
            self.dense.append(name)

    rec = Recorder()
    staf.load_into_store(rec, f)
    assert sorted(rec.f32) == ["model.layers.0.linear_attn.A_log", norm]
    assert np.array_equal(rec.f32["model.layers.0.linear_attn.A_log"], weights["model.layers.0.linear_attn.A_log"])
    assert "model.layers.0.linear_attn.dt_bias" in rec.dense and "model.layers.0.linear_attn.conv1d.weight" in rec.dense


def test_many_tensors_long_names_edge_values_and_shards(pkg, staf, tmp_path):
    """File-level properties of the reference's STAFDeepTests (Tests/MetalCompilerTests/Core/STAFDeepTests.swift:222-290
    '100 tensors load at non-overlapping offsets', :703-745 'payload starts at 256-byte aligned offset', :746-791 'shapes
    survive', :792-846 'Float16 edge values survive', :847-913 'Multiple safetensors shards merge', :958-996 'Long tensor
    names survive'), on this package's converter, writer and reader."""
    rng = np.random.default_rng(3)
    edge = np.array([0.0, -0.0, 65504.0, -65504.0, 6.1035e-05, 5.96e-08, 1.0, -1.0], dtype=np.float16)
    long_name = "model.layers.0." + ".".join(f"block{i}" for i in range(40)) + ".weight"
    shards = []
    for shard in range(2):
        tensors = {}
        for i in range(50):
            shape = (1 + (i % 5), 3 + (i % 7))
            tensors[f"s{shard}.t{i:03d}.weight"] = ("F16", rng.normal(size=shape).astype(np.float16))
        tensors[f"s{shard}.edge.weight"] = ("F16", edge.reshape(2, 4))
        if shard == 1:
            tensors[long_name] = ("BF16", pkg.f32_to_bf16(rng.normal(size=(3, 5)).astype(np.float32)))
        path = os.path.join(tmp_path, f"model-0000{shard + 1}-of-00002.safetensors")
        staf.write_safetensors(path, tensors)
        shards.append((path, tensors))
    out = os.path.join(tmp_path, "model.staf")
    assert staf.convert_safetensors([p for p, _ in shards], out) is True
    f = staf.read_staf(out)
    assert len(f.names()) == 2 * 51 + 1 and f.metadata[staf.KEY_SOURCE_SHARD_COUNT] == 2
    spans = sorted((f[n].payload_offset, f[n].payload_size) for n in f.names())
    assert spans[0][0] % 4096 == 0
    for (o0, s0), (o1, _) in zip(spans, spans[1:]):
        assert o0 % 256 == 0 and o1 % 256 == 0 and o0 + s0 <= o1           # aligned, in order, no overlap
    for shard, (_, tensors) in enumerate(shards):
        for name, (_, arr) in tensors.items():
            e = f[name]
            assert e.shape == arr.shape and e.shard_index == shard
            assert bytes(f.payload(name)) == np.ascontiguousarray(arr).tobytes()   # bit patterns: -0, subnormals, max
    assert long_name in f.names() and len(long_name) > 300


def test_tensor_names_are_canonicalized_at_conversion(pkg, staf, golden, tmp_path):
    """TensorNameCanonicalizerTests (Tests/MetalCompilerTests/Core/TensorNameCanonicalizerTests.swift:7-86): identity,
    the MLX vision-language prefix rewritten to the HuggingFace form, other names untouched, detection from any one name,
    first rule wins; and the converter applies it before it pairs a weight with its scales and biases."""
    C = staf.TensorNameCanonicalizer
    for name in ("model.language_model.embed_tokens.weight", "model.visual.patch_embed.weight", "lm_head.weight"):
        assert staf.IDENTITY_NAMES.canonicalize(name) == name
    mlx = staf.MLX_VLM_TO_HUGGINGFACE
    assert mlx.canonicalize("language_model.model.embed_tokens.weight") == "model.language_model.embed_tokens.weight"
    assert mlx.canonicalize("language_model.model.layers.0.self_attn.q_proj.scales") == "model.language_model.layers.0.self_attn.q_proj.scales"
    for name in ("visual.blocks.0.attn.qkv.weight", "lm_head.weight", "model.language_model.embed_tokens.weight"):
        assert mlx.canonicalize(name) == name
    assert C.detect(["visual.x", "language_model.model.embed_tokens.weight"]) == mlx
    assert C.detect(["model.language_model.embed_tokens.weight", "model.visual.patch_embed.weight"]) == staf.IDENTITY_NAMES
    assert C.detect(["model.embed_tokens.weight", "lm_head.weight"]) == staf.IDENTITY_NAMES
    assert C((("a.", "x."), ("a.b.", "y."))).canonicalize("a.b.c") == "x.b.c"
    g = golden["gemv_multi_row"]
    w = pkg.pack_mlx_q4(np.array(g["q"], dtype=np.uint8))
    src = os.path.join(tmp_path, "model.safetensors")
    staf.write_safetensors(src, {
        "language_model.model.layers.0.mlp.down_proj.weight": ("U32", w),
        "language_model.model.layers.0.mlp.down_proj.scales": ("BF16", _bf(pkg, g["scales"])),
        "language_model.model.layers.0.mlp.down_proj.biases": ("BF16", _bf(pkg, g["zeros"])),
        "visual.patch_embed.weight": ("BF16", _bf(pkg, np.ones((2, 4)))),
    })
    out = os.path.join(tmp_path, "model.staf")
    staf.convert_safetensors([src], out)
    f = staf.read_staf(out)
    assert f.names() == ["model.language_model.layers.0.mlp.down_proj.weight", "visual.patch_embed.weight"]
    assert f["model.language_model.layers.0.mlp.down_proj.weight"].scheme == staf.SCHEME_Q4_G64


def test_bundle_metadata_carries_provenance(pkg, staf, tmp_path):
    """STAFModelBundleMetadataBuilderTests 'Builder emits provenance and prefers chat_template.jinja'
    (Tests/MetalCompilerTests/Core/STAFModelBundleMetadataBuilderTests.swift:8-58), on the same files; the hash is FNV-1a
    64 (STAFStableHash.swift), checked on its published test vectors; and a cache written with this metadata is valid
    for the bundle until one of the hashed files changes."""
    assert staf.stable_hash64(b"") == 0xcbf29ce484222325 and staf.stable_hash64(b"a") == 0xaf63dc4c8601ec8c
    assert staf.stable_hash64("foobar") == 0x85944171f73967e8
    assert staf.stable_hash64("ab", 1) == staf.stable_hash64(b"ab" + (1).to_bytes(8, "little"))
    d = str(tmp_path)
    files = {"config.json": b'{"model_type":"lfm2","hidden_size":2048}', "tokenizer.json": b'{"version":"1.0"}',
             "tokenizer_config.json": b'{"chat_template":"from tokenizer config"}', "special_tokens_map.json": b'{"eos_token":"<eos>"}',
             "chat_template.jinja": b"from jinja", "model.safetensors": bytes([0, 1, 2, 3])}
    for name, data in files.items():
        open(os.path.join(d, name), "wb").write(data)
    cfg = pkg.ModelConfig("lfm2", hidden=2048, intermediate=6144, layers=24, heads=16, kv_heads=8, head_dim=128, vocab=32768,
                          max_seq=64, attention_layers=(2, 5), tie_embeddings=True)
    shard = os.path.join(d, "model.safetensors")
    m = staf.bundle_metadata(d, "lfm2", cfg, files["config.json"], [shard])
    assert m[staf.KEY_SOURCE_FORMAT] == "safetensors" and m[staf.KEY_SOURCE_SHARD_COUNT] == 1
    assert m[staf.KEY_CONVERTER_VERSION] == staf.U32(staf.CONVERTER_VERSION) and m[staf.KEY_METADATA_SCHEMA_VERSION] == staf.U32(staf.METADATA_SCHEMA_VERSION)
    assert (m[staf.KEY_MODEL_FAMILY], m[staf.KEY_MODEL_HIDDEN], m[staf.KEY_MODEL_LAYERS]) == ("lfm2", 2048, 24)
    assert (m[staf.KEY_MODEL_INTERMEDIATE], m[staf.KEY_MODEL_VOCAB], m[staf.KEY_MODEL_HEADS], m[staf.KEY_MODEL_KV_HEADS]) == (6144, 32768, 16, 8)
    assert m[staf.KEY_MODEL_TIED] is True and m[staf.KEY_MODEL_HEAD_DIM] == 128 and isinstance(m[staf.KEY_MODEL_ROPE_THETA], float)
    assert all(m[k] is True for k in (staf.KEY_SRC_TOKENIZER_PRESENT, staf.KEY_SRC_TOKENIZER_CONFIG_PRESENT,
                                      staf.KEY_SRC_SPECIAL_TOKENS_PRESENT, staf.KEY_SRC_CHAT_TEMPLATE_PRESENT))
    assert m[staf.KEY_SRC_CHAT_TEMPLATE_SOURCE] == "chat_template.jinja"
    assert m[staf.KEY_SRC_CHAT_TEMPLATE_HASH] == staf.stable_hash64(b"from jinja")
    assert m[staf.KEY_SRC_CONFIG_HASH] == staf.stable_hash64(files["config.json"])
    for key in (staf.KEY_SRC_TOKENIZER_HASH, staf.KEY_SRC_TOKENIZER_CONFIG_HASH, staf.KEY_SRC_SPECIAL_TOKENS_HASH, staf.KEY_SRC_MANIFEST_HASH):
        assert isinstance(m[key], int) and 0 <= m[key] < 1 << 64
    # without chat_template.jinja the template of tokenizer_config.json is the one that counts
    os.remove(os.path.join(d, "chat_template.jinja"))
    m2 = staf.bundle_metadata(d, "lfm2", cfg, files["config.json"], [shard])
    assert m2[staf.KEY_SRC_CHAT_TEMPLATE_SOURCE] == "tokenizer_config.json"
    assert m2[staf.KEY_SRC_CHAT_TEMPLATE_HASH] == staf.stable_hash64(b"from tokenizer config")
    # a cache written with the bundle's metadata: valid for it, stale once config.json changes
    src = os.path.join(d, "w.safetensors")
    staf.write_safetensors(src, {"model.norm.weight": ("BF16", _bf(pkg, np.ones(8)))})
    expect = staf.bundle_metadata(d, "lfm2", cfg, files["config.json"], [src])
    out = os.path.join(d, "model.staf")
    assert staf.convert_safetensors([src], out, extra_metadata=expect) is True
    assert staf.is_valid(out, [src], expect)
    changed = staf.bundle_metadata(d, "lfm2", cfg, files["config.json"] + b" ", [src])
    assert not staf.is_valid(out, [src], changed)
