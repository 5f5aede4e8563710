"""STAF files on the host: read, validate, write, convert from MLX safetensors, and feed a weight store.

STAF is the reference's executable weight cache (Sources/MetalCompiler/STAF/STAFFormat.swift:52-167): a packed
64-byte header, 128-byte section entries, 32-byte metadata entries, a string table, then payloads (the first one on a
4096-byte boundary, every tensor on a 256-byte boundary). This module mirrors

  * `STAFLoader.load` (STAF/STAFLoader.swift:64-153): header + section table + names -> tensor entries;
  * `STAFWriter.write` (STAF/STAFWriter.swift:11-130): the same layout, metadata keys sorted, strings de-duplicated;
  * `STAFValidator.isValid` (STAF/STAFValidator.swift:5-80): magic, format version, table bounds, expected metadata
    contained, not older than its sources;
  * `STAFConversionPlanner` / `STAFPayloadConverter` for the tensors of the hot path: MLX 4-bit group-64 triples
    (`*.weight` u32, `*.scales`, `*.biases`) -> interleaved 36-byte blocks (scheme 0x40), dense bf16 / fp16 / fp32
    tensors stored row-major (0x01 / 0x00 / 0x02).

Nothing here touches a GPU; `load_into_store` hands the payloads to the C ABI (`swlm_weights_add_q4g64_staf`,
`swlm_weights_add_dense_bf16`).
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple, Union

import numpy as np

from .formats import bf16_to_f32, f32_to_bf16, repack_mlx_to_staf

MAGIC = 0x46415453                # "STAF", little-endian (STAFFormat.swift:13)
FORMAT_VERSION = 2                # STAFFormat.swift:27
METADATA_SCHEMA_VERSION = 1       # STAFFormat.swift:33
CONVERTER_VERSION = 3             # STAFFormat.swift:50
HEADER_SIZE, SECTION_ENTRY_SIZE, METADATA_ENTRY_SIZE = 64, 128, 32   # STAFFormat.swift:53-59
PAYLOAD_ALIGNMENT, TENSOR_ALIGNMENT, MAX_DIMS = 4096, 256, 8         # STAFFormat.swift:62-68

# QuantizationSchemeIdentifier (STAFFormat.swift:166-214), the ones this path stores or recognises
SCHEME_FP16, SCHEME_BF16, SCHEME_FP32 = 0x00, 0x01, 0x02
SCHEME_Q4_G64, SCHEME_Q4_G128 = 0x40, 0x41
SCHEME_PASSTHROUGH = 0xFF
# SemanticRole (STAFFormat.swift:282-299)
ROLE_UNKNOWN, ROLE_TOKEN_EMBEDDING, ROLE_Q, ROLE_K, ROLE_V, ROLE_O = 0x00, 0x01, 0x02, 0x03, 0x04, 0x05
ROLE_GATE, ROLE_UP, ROLE_DOWN, ROLE_NORM, ROLE_LM_HEAD, ROLE_OTHER = 0x06, 0x07, 0x08, 0x09, 0x0A, 0xFF
# OriginalDType (STAFFormat.swift:304-313)
DTYPE_F32, DTYPE_F16, DTYPE_BF16, DTYPE_I32, DTYPE_UNKNOWN = 0x00, 0x01, 0x02, 0x03, 0xFF
# STAFMetadataValueType (STAFMetadataValue.swift:12-19)
MV_BOOL, MV_U32, MV_U64, MV_F32, MV_F64, MV_STRING = 0x01, 0x02, 0x03, 0x04, 0x05, 0x06

# STAFMetadataKey.swift
KEY_SOURCE_FORMAT = "general.source_format"
KEY_CONVERTER_VERSION = "staf.converter_version"
KEY_SOURCE_SHARD_COUNT = "staf.source_shard_count"
KEY_METADATA_SCHEMA_VERSION = "staf.metadata_schema_version"


# model and provenance keys of a bundle's cache (STAFMetadataKey.swift:9-34)
KEY_MODEL_FAMILY, KEY_MODEL_HIDDEN, KEY_MODEL_LAYERS = "model.architecture_family", "model.hidden_size", "model.layer_count"
KEY_MODEL_INTERMEDIATE, KEY_MODEL_VOCAB = "model.intermediate_size", "model.vocab_size"
KEY_MODEL_HEADS, KEY_MODEL_KV_HEADS, KEY_MODEL_HEAD_DIM = "model.attention_heads", "model.kv_heads", "model.head_dim"
KEY_MODEL_TIED, KEY_MODEL_ROPE_DIM, KEY_MODEL_ROPE_THETA = "model.tied_embeddings", "model.rope_dimension", "model.rope_theta"
KEY_SRC_CONFIG_HASH, KEY_SRC_MANIFEST_HASH = "source.config_hash", "source.safetensors_manifest_hash"
KEY_SRC_TOKENIZER_HASH, KEY_SRC_TOKENIZER_CONFIG_HASH = "source.tokenizer_hash", "source.tokenizer_config_hash"
KEY_SRC_SPECIAL_TOKENS_HASH, KEY_SRC_CHAT_TEMPLATE_HASH = "source.special_tokens_hash", "source.chat_template_hash"
KEY_SRC_CHAT_TEMPLATE_SOURCE = "source.chat_template_source"
KEY_SRC_TOKENIZER_PRESENT, KEY_SRC_TOKENIZER_CONFIG_PRESENT = "source.tokenizer_present", "source.tokenizer_config_present"
KEY_SRC_SPECIAL_TOKENS_PRESENT, KEY_SRC_CHAT_TEMPLATE_PRESENT = "source.special_tokens_present", "source.chat_template_present"
CHAT_TEMPLATE_JINJA_SOURCE, TOKENIZER_CONFIG_SOURCE = "chat_template.jinja", "tokenizer_config.json"


class STAFError(ValueError):
    pass


@dataclass(frozen=True)
class U32:
    """A metadata value stored as uint32 (plain Python ints are stored as uint64)."""
    value: int


@dataclass(frozen=True)
class F32:
    """A metadata value stored as float32 (plain Python floats are stored as float64)."""
    value: float


MetadataValue = Union[bool, int, float, str, U32, F32]


@dataclass
class TensorEntry:
    """One section: STAFTensorEntry of the reference's loader plus the fields the writer stores."""
    name: str
    scheme: int
    role: int
    original_dtype: int
    shape: Tuple[int, ...]
    payload_offset: int
    payload_size: int
    alignment: int = TENSOR_ALIGNMENT
    block_size: int = 1
    group_size: int = 1
    checksum: int = 0
    shard_index: int = 0


@dataclass
class STAFFile:
    path: str
    format_version: int
    entries: List[TensorEntry]
    metadata: Dict[str, MetadataValue]
    data: np.ndarray = field(repr=False)   # the whole file, memory-mapped, uint8

    def __getitem__(self, name: str) -> TensorEntry:
        for e in self.entries:
            if e.name == name:
                return e
        raise KeyError(name)

    def names(self) -> List[str]:
        return [e.name for e in self.entries]

    def payload(self, name: str) -> np.ndarray:
        e = self[name]
        return self.data[e.payload_offset:e.payload_offset + e.payload_size]


def default_cache_metadata(source_shard_count: int) -> Dict[str, MetadataValue]:
    """STAFFileMetadata.defaultCacheMetadata (STAF/STAFFileMetadata.swift:50-58)."""
    return {KEY_SOURCE_FORMAT: "safetensors", KEY_CONVERTER_VERSION: U32(CONVERTER_VERSION),
            KEY_SOURCE_SHARD_COUNT: int(source_shard_count), KEY_METADATA_SCHEMA_VERSION: U32(METADATA_SCHEMA_VERSION)}


def stable_hash64(*parts: Union[bytes, str, int]) -> int:
    """STAFStableHash64 (STAFStableHash.swift:3-42): FNV-1a over the bytes of every part in order; a string enters as
    UTF-8, an integer as 8 little-endian bytes."""
    state = 0xcbf29ce484222325
    for part in parts:
        data = part.encode() if isinstance(part, str) else struct.pack("<Q", part) if isinstance(part, int) else bytes(part)
        for byte in data:
            state = ((state ^ byte) * 0x00000100000001B3) & 0xFFFFFFFFFFFFFFFF
    return state


def bundle_metadata(directory: str, model_type: str, config, config_data: bytes, safetensors_paths: Sequence[str]) -> Dict[str, MetadataValue]:
    """What a bundle's STAF cache must carry to be taken as valid for that bundle (STAFModelBundleMetadataBuilder.swift:
    7-128): the model's dimensions (`config`: a plan.ModelConfig), which tokenizer files are present, FNV-1a hashes of
    config.json, of the tokenizer files and of the chat template (chat_template.jinja wins over the `chat_template` string
    of tokenizer_config.json), and a hash over (file name, size, modification time in ns) of the shards sorted by name;
    merged over the converter's own keys."""
    def optional(name):
        path = os.path.join(directory, name)
        return open(path, "rb").read() if os.path.exists(path) else None

    tokenizer, tokenizer_config, special = optional("tokenizer.json"), optional("tokenizer_config.json"), optional("special_tokens_map.json")
    template = optional("chat_template.jinja")
    template_source = CHAT_TEMPLATE_JINJA_SOURCE if template is not None else None
    if template is None and tokenizer_config is not None:
        parsed = json.loads(tokenizer_config.decode())
        if isinstance(parsed, dict) and isinstance(parsed.get("chat_template"), str):
            template, template_source = parsed["chat_template"].encode(), TOKENIZER_CONFIG_SOURCE
    values: Dict[str, MetadataValue] = {
        KEY_MODEL_FAMILY: model_type, KEY_MODEL_HIDDEN: int(config.hidden), KEY_MODEL_LAYERS: int(config.layers),
        KEY_MODEL_INTERMEDIATE: int(config.intermediate), KEY_MODEL_VOCAB: int(config.vocab), KEY_MODEL_HEADS: int(config.heads),
        KEY_MODEL_KV_HEADS: int(config.kv_heads), KEY_MODEL_HEAD_DIM: int(config.head_dim),
        KEY_MODEL_TIED: bool(config.tie_embeddings), KEY_MODEL_ROPE_DIM: int(config.head_dim),
        KEY_MODEL_ROPE_THETA: float(config.rope_theta),
        KEY_SRC_TOKENIZER_PRESENT: tokenizer is not None, KEY_SRC_TOKENIZER_CONFIG_PRESENT: tokenizer_config is not None,
        KEY_SRC_SPECIAL_TOKENS_PRESENT: special is not None, KEY_SRC_CHAT_TEMPLATE_PRESENT: template is not None,
        KEY_SRC_CONFIG_HASH: stable_hash64(config_data),
    }
    manifest = []
    for path in sorted(safetensors_paths, key=os.path.basename):
        st = os.stat(os.path.realpath(path))
        manifest += [os.path.basename(path), int(st.st_size), max(0, int(st.st_mtime_ns))]
    values[KEY_SRC_MANIFEST_HASH] = stable_hash64(*manifest)
    for key, data in ((KEY_SRC_TOKENIZER_HASH, tokenizer), (KEY_SRC_TOKENIZER_CONFIG_HASH, tokenizer_config),
                      (KEY_SRC_SPECIAL_TOKENS_HASH, special), (KEY_SRC_CHAT_TEMPLATE_HASH, template)):
        if data is not None:
            values[key] = stable_hash64(data)
    if template_source is not None:
        values[KEY_SRC_CHAT_TEMPLATE_SOURCE] = template_source
    merged = default_cache_metadata(len(safetensors_paths))
    merged.update(values)
    return merged


def _align_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


# ---- reading -------------------------------------------------------------------------------------------------

def read_staf(path: str) -> STAFFile:
    """Parse header, section table, string table and metadata table; payloads stay memory-mapped."""
    size = os.path.getsize(path)
    if size < HEADER_SIZE:
        raise STAFError("file shorter than the 64-byte header")
    data = np.memmap(path, dtype=np.uint8, mode="r")
    head = bytes(data[:HEADER_SIZE])
    magic, version, meta_count, meta_off = struct.unpack_from("<IIII", head, 0)
    section_count, section_off, string_off, string_size = struct.unpack_from("<IIII", head, 40)
    if magic != MAGIC:
        raise STAFError(f"bad magic {magic:#x}")
    if section_off + section_count * SECTION_ENTRY_SIZE > size or string_off + string_size > size:
        raise STAFError("section or string table outside the file")
    strings = bytes(data[string_off:string_off + string_size])

    def text(offset: int, length: int) -> str:
        if offset + length > len(strings):
            raise STAFError("string outside the string table")
        return strings[offset:offset + length].decode("utf-8", "replace")

    entries = []
    for i in range(section_count):
        base = bytes(data[section_off + i * SECTION_ENTRY_SIZE:section_off + (i + 1) * SECTION_ENTRY_SIZE])
        name_off, name_len, scheme, role, odt, ndim = struct.unpack_from("<IIBBBB", base, 0)
        shape = struct.unpack_from("<8I", base, 12)[:min(ndim, MAX_DIMS)]
        p_off, p_size = struct.unpack_from("<QQ", base, 44)
        align, block, group, crc, shard = struct.unpack_from("<IIIII", base, 60)
        if p_off > size or p_size > size or p_off + p_size > size:
            raise STAFError(f"payload of section {i} outside the file")
        entries.append(TensorEntry(text(name_off, name_len), scheme, role, odt, tuple(int(d) for d in shape), int(p_off),
                                   int(p_size), int(align), int(block), int(group), int(crc), int(shard)))
    if not entries:
        raise STAFError("no tensors in STAF")
    metadata: Dict[str, MetadataValue] = {}
    if version >= FORMAT_VERSION and meta_count > 0 and meta_off > 0:   # STAFHeader.supportsMetadataTable
        if meta_off < HEADER_SIZE + section_count * SECTION_ENTRY_SIZE or meta_off + meta_count * METADATA_ENTRY_SIZE > size:
            raise STAFError("metadata table outside the file")
        for i in range(meta_count):
            base = bytes(data[meta_off + i * METADATA_ENTRY_SIZE:meta_off + (i + 1) * METADATA_ENTRY_SIZE])
            key_off, key_len, vtype = struct.unpack_from("<IIB", base, 0)
            p0, p1 = struct.unpack_from("<QQ", base, 12)
            key = text(key_off, key_len)
            if vtype == MV_BOOL:
                metadata[key] = bool(p0)
            elif vtype == MV_U32:
                metadata[key] = U32(int(p0))
            elif vtype == MV_U64:
                metadata[key] = int(p0)
            elif vtype == MV_F32:
                metadata[key] = F32(struct.unpack("<f", struct.pack("<I", p0 & 0xFFFFFFFF))[0])
            elif vtype == MV_F64:
                metadata[key] = struct.unpack("<d", struct.pack("<Q", p0))[0]
            elif vtype == MV_STRING:
                metadata[key] = text(int(p0), int(p1))
            else:
                raise STAFError(f"metadata '{key}': unknown value type {vtype}")
    return STAFFile(path, int(version), entries, metadata, data)


def is_valid(path: str, source_paths: Sequence[str] = (), expected_metadata: Optional[Dict[str, MetadataValue]] = None) -> bool:
    """STAFValidator.isValid: current format version, section table right behind the header, tables and first payload
    inside the file, every expected metadata value present and equal, and the cache not older than any source."""
    try:
        size = os.path.getsize(path)
        if size < HEADER_SIZE:
            return False
        with open(path, "rb") as f:
            head = f.read(HEADER_SIZE + SECTION_ENTRY_SIZE)
        magic, version, _, _ = struct.unpack_from("<IIII", head, 0)
        section_count, section_off = struct.unpack_from("<II", head, 40)
        if magic != MAGIC or section_count == 0 or version != FORMAT_VERSION or section_off != HEADER_SIZE:
            return False
        if size > HEADER_SIZE + SECTION_ENTRY_SIZE and struct.unpack_from("<Q", head, HEADER_SIZE + 52)[0] > size:
            return False
        staf = read_staf(path)
    except (OSError, STAFError, struct.error):
        return False
    if expected_metadata:
        for key, want in expected_metadata.items():
            if key not in staf.metadata or staf.metadata[key] != want:
                return False
    mtime = os.path.getmtime(path)
    for src in source_paths:
        if os.path.getmtime(os.path.realpath(src)) > mtime:
            return False
    return True


# ---- writing -------------------------------------------------------------------------------------------------

@dataclass
class TensorToWrite:
    """What STAFWriter needs of a STAFConversionEntry: the section's fields and the converted payload. `shape` is the
    source safetensors shape (for a quantized tensor the packed one, [n, k/8] words)."""
    name: str
    scheme: int
    role: int
    original_dtype: int
    shape: Tuple[int, ...]
    payload: bytes
    block_size: int = 1
    group_size: int = 1
    shard_index: int = 0


def _metadata_entry(key: str, value: MetadataValue, key_off: int, intern) -> bytes:
    if isinstance(value, bool):
        vtype, p0, p1 = MV_BOOL, int(value), 0
    elif isinstance(value, U32):
        vtype, p0, p1 = MV_U32, value.value & 0xFFFFFFFF, 0
    elif isinstance(value, int):
        vtype, p0, p1 = MV_U64, value, 0
    elif isinstance(value, F32):
        vtype, p0, p1 = MV_F32, struct.unpack("<I", struct.pack("<f", value.value))[0], 0
    elif isinstance(value, float):
        vtype, p0, p1 = MV_F64, struct.unpack("<Q", struct.pack("<d", value))[0], 0
    elif isinstance(value, str):
        vtype, p0, p1 = MV_STRING, intern(value), len(value.encode())
    else:
        raise STAFError(f"metadata '{key}': unsupported value {value!r}")
    out = bytearray(METADATA_ENTRY_SIZE)
    struct.pack_into("<IIB", out, 0, key_off, len(key.encode()), vtype)
    struct.pack_into("<QQ", out, 12, p0, p1)
    return bytes(out)


def write_staf(path: str, tensors: Sequence[TensorToWrite], metadata: Optional[Dict[str, MetadataValue]] = None) -> None:
    """STAFWriter.write: header | section table | metadata table (keys sorted) | string table (tensor names in order,
    then metadata keys and string values, each stored once, NUL-terminated) | payloads (first on 4096, each on 256)."""
    metadata = dict(metadata or {})
    strings = bytearray()
    offsets: Dict[str, int] = {}

    def intern(s: str) -> int:
        if s in offsets:
            return offsets[s]
        off = len(strings)
        strings.extend(s.encode())
        strings.append(0)
        offsets[s] = off
        return off

    name_offsets = [intern(t.name) for t in tensors]
    meta_entries = []
    for key in sorted(metadata):
        key_off = intern(key)
        meta_entries.append(_metadata_entry(key, metadata[key], key_off, intern))
    section_off = HEADER_SIZE
    meta_off = section_off + len(tensors) * SECTION_ENTRY_SIZE
    string_off = meta_off + len(meta_entries) * METADATA_ENTRY_SIZE
    payload_start = _align_up(string_off + len(strings), PAYLOAD_ALIGNMENT)
    payload_offsets, cur = [], payload_start
    for t in tensors:
        at = _align_up(cur, TENSOR_ALIGNMENT)
        payload_offsets.append(at)
        cur = at + len(t.payload)

    head = bytearray(HEADER_SIZE)
    struct.pack_into("<IIII", head, 0, MAGIC, FORMAT_VERSION, len(meta_entries), meta_off)
    struct.pack_into("<IIII", head, 40, len(tensors), section_off, string_off, len(strings))
    with open(path, "wb") as f:
        f.write(head)
        for t, name_off, p_off in zip(tensors, name_offsets, payload_offsets):
            e = bytearray(SECTION_ENTRY_SIZE)
            ndim = min(len(t.shape), MAX_DIMS)
            struct.pack_into("<IIBBBB", e, 0, name_off, len(t.name.encode()), t.scheme, t.role, t.original_dtype, ndim)
            struct.pack_into("<8I", e, 12, *(list(t.shape[:ndim]) + [0] * (MAX_DIMS - ndim)))
            struct.pack_into("<QQ", e, 44, p_off, len(t.payload))
            struct.pack_into("<IIIII", e, 60, TENSOR_ALIGNMENT, t.block_size, t.group_size, 0, t.shard_index)
            f.write(e)
        for m in meta_entries:
            f.write(m)
        f.write(strings)
        pos = string_off + len(strings)
        for t, p_off in zip(tensors, payload_offsets):
            if pos < p_off:
                f.write(b"\0" * (p_off - pos))
            f.write(t.payload)
            pos = p_off + len(t.payload)


# ---- MLX safetensors -> STAF ----------------------------------------------------------------------------------

_ST_DTYPES = {"F32": (np.float32, DTYPE_F32), "F16": (np.float16, DTYPE_F16), "BF16": (np.uint16, DTYPE_BF16),
              "U32": (np.uint32, DTYPE_I32), "I32": (np.int32, DTYPE_I32)}


def read_safetensors(path: str) -> Dict[str, Tuple[str, Tuple[int, ...], np.ndarray]]:
    """name -> (dtype string, shape, array). The file is an 8-byte little-endian header length, a JSON header
    {name: {dtype, shape, data_offsets}}, then the tensor bytes. bf16 tensors come back as uint16 bit patterns."""
    data = np.memmap(path, dtype=np.uint8, mode="r")
    (hlen,) = struct.unpack("<Q", bytes(data[:8]))
    header = json.loads(bytes(data[8:8 + hlen]).decode())
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        if info["dtype"] not in _ST_DTYPES:
            raise STAFError(f"{name}: dtype {info['dtype']} is outside the hot path")
        np_dtype = _ST_DTYPES[info["dtype"]][0]
        lo, hi = info["data_offsets"]
        out[name] = (info["dtype"], tuple(info["shape"]), np.frombuffer(data[8 + hlen + lo:8 + hlen + hi], dtype=np_dtype).reshape(info["shape"]))
    return out


def safetensors_names(path: str) -> List[str]:
    """Tensor names of a shard, from its JSON header alone."""
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen).decode())
    return [name for name in header if name != "__metadata__"]


def write_safetensors(path: str, tensors: Dict[str, Tuple[str, np.ndarray]]) -> None:
    """Minimal writer (tests build MLX-shaped bundles with it): name -> (dtype string, array)."""
    header, blobs, off = {}, [], 0
    for name, (dtype, arr) in tensors.items():
        raw = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def semantic_role(name: str) -> int:
    """Role hint from the canonical tensor name (the runtime does not depend on it)."""
    table = (("embed_tokens", ROLE_TOKEN_EMBEDDING), ("lm_head", ROLE_LM_HEAD), ("q_proj", ROLE_Q), ("k_proj", ROLE_K),
             ("v_proj", ROLE_V), ("o_proj", ROLE_O), ("out_proj", ROLE_O), ("gate_proj", ROLE_GATE), ("w1", ROLE_GATE),
             ("up_proj", ROLE_UP), ("w3", ROLE_UP), ("down_proj", ROLE_DOWN), ("w2", ROLE_DOWN), ("norm", ROLE_NORM))
    for key, role in table:
        if key in name:
            return role
    return ROLE_OTHER


@dataclass(frozen=True)
class TensorNameCanonicalizer:
    """Source-convention tensor names into the HuggingFace form the naming conventions expect
    (STAF/TensorNameCanonicalizer.swift:15-77): prefix-substitution rules, the first match wins. MLX vision-language
    bundles package the text backbone under `language_model.model.*` where HuggingFace has `model.language_model.*`."""
    rules: Tuple[Tuple[str, str], ...] = ()

    def canonicalize(self, name: str) -> str:
        for src, dst in self.rules:
            if name.startswith(src):
                return dst + name[len(src):]
        return name

    @staticmethod
    def detect(names: Iterable[str]) -> "TensorNameCanonicalizer":
        """The MLX rule when any name carries the MLX prefix (the two conventions exclude each other), else identity."""
        for name in names:
            if name.startswith("language_model.model."):
                return MLX_VLM_TO_HUGGINGFACE
        return IDENTITY_NAMES


IDENTITY_NAMES = TensorNameCanonicalizer()
MLX_VLM_TO_HUGGINGFACE = TensorNameCanonicalizer((("language_model.model.", "model.language_model."),))


def plan_conversion(tensors: Dict[str, Tuple[str, Tuple[int, ...], np.ndarray]], bits: int = 4, group_size: int = 64,
                    shard_index: int = 0) -> List[TensorToWrite]:
    """STAFConversionPlanner + STAFPayloadConverter for one shard: a `*.weight` with `.scales` and `.biases` companions
    is an MLX quantized triple (the companions are consumed, STAFConversionPlanner.swift:63-78) and becomes interleaved
    blocks (36 bytes for group 64, scheme 0x40; 68 bytes for group 128, scheme 0x41); every other tensor is stored
    row-major in its own dtype. Entries keep the source order. `bits` / `group_size` are the bundle's quantization hint
    (config.json `quantization`), checked against the tensor shapes as STAFConversionPlanner.verifyTensorShape does."""
    if bits != 4 or group_size not in (64, 128):
        raise STAFError(f"MLX quantization bits={bits} group_size={group_size} is outside the hot path (4-bit, group 64 or 128)")
    consumed = set()
    for name in tensors:
        if name.endswith(".weight"):
            mod = name[:-len(".weight")]
            if mod + ".scales" in tensors and mod + ".biases" in tensors:
                consumed.update((mod + ".scales", mod + ".biases"))
    out = []
    for name, (dtype, shape, arr) in tensors.items():
        if name in consumed:
            continue
        mod = name[:-len(".weight")] if name.endswith(".weight") else None
        if mod is not None and mod + ".scales" in consumed:
            scales, biases = tensors[mod + ".scales"], tensors[mod + ".biases"]
            n, words = shape
            k = words * 32 // bits
            if scales[1] != (n, k // group_size) or biases[1] != (n, k // group_size) or dtype != "U32":
                raise STAFError(f"{name}: shapes of the quantized triple disagree")

            def as_bf16(t):
                return t[2] if t[0] == "BF16" else f32_to_bf16(np.asarray(t[2], dtype=np.float32))

            blocks = repack_mlx_to_staf(np.asarray(arr), as_bf16(scales), as_bf16(biases), group=group_size)
            out.append(TensorToWrite(name, SCHEME_Q4_G64 if group_size == 64 else SCHEME_Q4_G128, semantic_role(name), DTYPE_I32,
                                     tuple(shape), blocks.tobytes(), block_size=group_size, group_size=group_size,
                                     shard_index=shard_index))
            continue
        if name.endswith(".linear_attn.norm.weight") and dtype in ("BF16", "F16"):
            # the recurrent layers' norm weight is read as fp32 by the kernel: promoted whatever the bundle stores
            # (STAFConversionPlanner.swift:117-127, isSSMNormWeight :138-140)
            f = bf16_to_f32(np.asarray(arr)) if dtype == "BF16" else np.asarray(arr).view(np.float16).astype(np.float32)
            out.append(TensorToWrite(name, SCHEME_FP32, semantic_role(name), _ST_DTYPES["F32"][1], tuple(shape),
                                     np.ascontiguousarray(f, dtype=np.float32).tobytes(), shard_index=shard_index))
            continue
        scheme = {"F16": SCHEME_FP16, "BF16": SCHEME_BF16, "F32": SCHEME_FP32}.get(dtype, SCHEME_PASSTHROUGH)
        out.append(TensorToWrite(name, scheme, semantic_role(name), _ST_DTYPES[dtype][1], tuple(shape),
                                 np.ascontiguousarray(arr).tobytes(), shard_index=shard_index))
    return out


def convert_safetensors(safetensors_paths: Sequence[str], staf_path: str, extra_metadata: Optional[Dict[str, MetadataValue]] = None,
                        force: bool = False, group_size: int = 64) -> bool:
    """Write `staf_path` from the shards unless a valid cache is already there (STAFConverter's
    convert-if-invalid). Returns True when the file was (re)written."""
    expected = default_cache_metadata(len(safetensors_paths))
    expected.update(extra_metadata or {})
    if not force and os.path.exists(staf_path) and is_valid(staf_path, safetensors_paths, expected):
        return False
    entries: List[TensorToWrite] = []
    shards = [read_safetensors(p) for p in sorted(safetensors_paths)]
    # the source convention is detected over all shards, and every name canonicalized before the quantized triples
    # are matched (STAFConversionPlanner.swift:21-31)
    names = TensorNameCanonicalizer.detect(n for t in shards for n in t)
    for shard, tensors in enumerate(shards):
        entries += plan_conversion({names.canonicalize(n): v for n, v in tensors.items()}, group_size=group_size, shard_index=shard)
    write_staf(staf_path, entries, expected)
    return True


# ---- into the weight store -------------------------------------------------------------------------------------

def load_into_store(store, staf: STAFFile, shard_kinds: Optional[Dict[str, int]] = None, names: Optional[Iterable[str]] = None) -> List[str]:
    """Hand every tensor of the file that the hot path can hold to the weight store: 4-bit group-64 / group-128 block
    tensors as they are (`swlm_weights_add_q4g64_staf`, `swlm_weights_add_q4g128_staf`), dense tensors as bf16 (fp16 and fp32 sources are rounded to bf16, the
    activation dtype of the path). `shard_kinds` maps names to SWLM_SHARD_* for tensor-parallel contexts. Returns the
    names loaded; tensors of other schemes are skipped."""
    shard_kinds = shard_kinds or {}
    wanted = set(names) if names is not None else None
    loaded = []
    for e in staf.entries:
        if wanted is not None and e.name not in wanted:
            continue
        raw = np.asarray(staf.data[e.payload_offset:e.payload_offset + e.payload_size])
        if e.scheme in (SCHEME_Q4_G64, SCHEME_Q4_G128):
            n, words = e.shape
            k = words * 8
            group = 64 if e.scheme == SCHEME_Q4_G64 else 128
            bb = 4 + group // 2
            if k % group or e.payload_size != n * (k // group) * bb:
                raise STAFError(f"{e.name}: payload size does not match {n} x {k} in {bb}-byte blocks")
            if group == 64:
                store.add_q4_staf(e.name, raw.reshape(n, k // 64, 36), n, k, shard_kinds.get(e.name, 0))
            else:
                store.add_q4_staf(e.name, raw.reshape(n, k // 128, 68), n, k, shard_kinds.get(e.name, 0), group=128)
        elif e.scheme == SCHEME_FP32 and (e.name.endswith(".linear_attn.norm.weight") or e.name.endswith(".A_log")) and hasattr(store, "add_dense_f32"):
            store.add_dense_f32(e.name, raw.view(np.float32))    # what the recurrent step reads as fp32 stays fp32
        elif e.scheme in (SCHEME_BF16, SCHEME_FP16, SCHEME_FP32, SCHEME_PASSTHROUGH):
            if e.scheme == SCHEME_BF16:
                arr = raw.view(np.uint16)
            elif e.scheme == SCHEME_FP32:
                arr = f32_to_bf16(raw.view(np.float32))
            else:
                arr = f32_to_bf16(raw.view(np.float16).astype(np.float32))
            shape = e.shape if len(e.shape) >= 1 else (1,)
            rows = int(np.prod(shape[:-1])) if len(shape) > 1 else 1
            store.add_dense(e.name, np.ascontiguousarray(arr).reshape(rows, shape[-1]), shard_kinds.get(e.name, 0))
        else:
            continue
        loaded.append(e.name)
    return loaded
