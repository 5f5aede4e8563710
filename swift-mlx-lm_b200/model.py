"""Host-side mirror of the reference's weight store and inference model over the C ABI.

`WeightStore` stands for `STAFWeightStore` (Sources/MetalCompiler/STAF/STAFLoader.swift:213-299) and
`InferenceModel` for `MetalInferenceModel` (Sources/MetalCompiler/Execution/MetalInferenceModel.swift:
prefill :464, decode :311, resetState :1911, promptSnapshot/restore :1897-1906, position :9).
Method names keep the reference's meaning; errors raise `SwlmError` where the reference throws, and a
failed decode returns token -1 as `MetalDecodeExecutor` does (Execution/MetalDecodeExecutor.swift:33-42).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from .lib import BuffersDesc, Library, Step, load_library


def _ptr(a: np.ndarray) -> C.c_void_p:
    return a.ctypes.data_as(C.c_void_p)


class WeightStore:
    def __init__(self, device: int = 0, tp_rank: int = 0, tp_size: int = 1, lib: Optional[Library] = None):
        self.lib = lib or load_library()
        self.handle = C.c_void_p()
        self.lib.check(self.lib.swlm_ctx_create(device, tp_rank, tp_size, C.byref(self.handle)))
        self.tp_rank, self.tp_size = tp_rank, tp_size

    def close(self) -> None:
        if self.handle:
            self.lib.swlm_ctx_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def add_q4_mlx(self, name: str, weight: np.ndarray, scales_bf16: np.ndarray, biases_bf16: np.ndarray, shard: int = 0) -> None:
        w = np.ascontiguousarray(weight, dtype=np.uint32)
        s = np.ascontiguousarray(scales_bf16, dtype=np.uint16)
        b = np.ascontiguousarray(biases_bf16, dtype=np.uint16)
        n, words = w.shape
        # the group size (64 or 128 weights per scale / bias pair) follows from the shape of the scales
        group = words * 8 // s.shape[-1] if s.size else 64
        if group not in (64, 128) or s.shape != (n, words * 8 // group) or b.shape != s.shape:
            raise ValueError(f"{name}: scales {s.shape} / biases {b.shape} do not describe groups of 64 or 128 over k={words * 8}")
        add = self.lib.swlm_weights_add_q4g64_mlx if group == 64 else self.lib.swlm_weights_add_q4g128_mlx
        self.lib.check(add(self.handle, name.encode(), n, words * 8, _ptr(w), _ptr(s), _ptr(b), shard))

    def add_q4_staf(self, name: str, blocks: np.ndarray, n: int, k: int, shard: int = 0, group: int = 64) -> None:
        blk = np.ascontiguousarray(blocks, dtype=np.uint8)
        if blk.size != n * (k // group) * (4 + group // 2):
            raise ValueError(f"{name}: {blk.size} bytes are not {n} x {k // group} blocks of {4 + group // 2} bytes")
        add = self.lib.swlm_weights_add_q4g64_staf if group == 64 else self.lib.swlm_weights_add_q4g128_staf
        self.lib.check(add(self.handle, name.encode(), n, k, _ptr(blk), shard))

    def add_dense_f32(self, name: str, data: np.ndarray) -> None:
        """fp32 tensor, replicated (norm weight and A_log of the recurrent layers)."""
        d = np.ascontiguousarray(data, dtype=np.float32)
        self.lib.check(self.lib.swlm_weights_add_dense_f32(self.handle, name.encode(), d.size, _ptr(d)))

    def add_dense(self, name: str, data_bf16: np.ndarray, shard: int = 0) -> None:
        d = np.ascontiguousarray(data_bf16, dtype=np.uint16)
        rows = d.shape[0] if d.ndim == 2 else 1
        cols = d.size // rows
        self.lib.check(self.lib.swlm_weights_add_dense_bf16(self.handle, name.encode(), rows, cols, _ptr(d), shard))

    @property
    def resident_bytes(self) -> int:
        return int(self.lib.swlm_weights_bytes(self.handle))

    # op-level entry points -----------------------------------------------------------------------
    def qgemm(self, name: str, x_bf16: np.ndarray, n: int) -> np.ndarray:
        x = np.ascontiguousarray(x_bf16, dtype=np.uint16)
        m = x.shape[0]
        y = np.empty((m, n), dtype=np.uint16)
        self.lib.check(self.lib.swlm_op_qgemm(self.handle, name.encode(), m, _ptr(x), _ptr(y)))
        return y

    def dequant_bf16(self, name: str, n: int, k: int) -> np.ndarray:
        out = np.empty((n, k), dtype=np.uint16)
        self.lib.check(self.lib.swlm_op_dequant_bf16(self.handle, name.encode(), _ptr(out)))
        return out


class InferenceModel:
    """Compiled plan + one isolated runtime state."""

    def __init__(self, store: WeightStore, steps: Sequence[Step], desc: BuffersDesc):
        self.store = store
        self.lib = store.lib
        self.desc = desc
        self.batch = int(desc.max_batch)
        arr = (Step * len(steps))(*steps)
        self.plan = C.c_void_p()
        self.lib.check(self.lib.swlm_plan_build(store.handle, arr, len(steps), C.byref(desc), C.byref(self.plan)))
        self.state = C.c_void_p()
        self.lib.check(self.lib.swlm_state_create(self.plan, C.byref(self.state)))

    def close(self) -> None:
        if getattr(self, "state", None):
            self.lib.swlm_state_destroy(self.state)
            self.state = C.c_void_p()
        if getattr(self, "plan", None):
            self.lib.swlm_plan_destroy(self.plan)
            self.plan = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- reference surface ---------------------------------------------------------------------------
    @property
    def position(self) -> int:
        return int(self.lib.swlm_position(self.state))

    def reset_state(self) -> None:
        self.lib.check(self.lib.swlm_state_reset(self.state))

    def prefill(self, tokens) -> np.ndarray:
        t = np.ascontiguousarray(np.atleast_2d(np.asarray(tokens, dtype=np.int32)))
        assert t.shape[0] == self.batch
        first = np.empty(self.batch, dtype=np.int32)
        self.lib.check(self.lib.swlm_prefill(self.state, _ptr(t), t.shape[1], _ptr(first)))
        return first

    def decode(self, token_in) -> np.ndarray:
        t = np.ascontiguousarray(np.asarray(token_in, dtype=np.int32).reshape(self.batch))
        out = np.empty(self.batch, dtype=np.int32)
        self.lib.check(self.lib.swlm_decode(self.state, _ptr(t), _ptr(out)))
        return out

    def decode_n(self, token_in, n: int) -> np.ndarray:
        t = np.ascontiguousarray(np.asarray(token_in, dtype=np.int32).reshape(self.batch))
        out = np.empty((n, self.batch), dtype=np.int32)
        self.lib.check(self.lib.swlm_decode_n(self.state, _ptr(t), n, _ptr(out)))
        return out

    def decode_n_async(self, token_in, n: int) -> None:
        p = None
        if token_in is not None:
            t = np.ascontiguousarray(np.asarray(token_in, dtype=np.int32).reshape(self.batch))
            p = _ptr(t)
        self.lib.check(self.lib.swlm_decode_n_async(self.state, p, n))

    def read_tokens(self, n: int) -> np.ndarray:
        out = np.empty((n, self.batch), dtype=np.int32)
        self.lib.check(self.lib.swlm_read_tokens(self.state, n, _ptr(out)))
        return out

    def sync(self) -> None:
        self.lib.check(self.lib.swlm_sync(self.state))

    def set_stream(self, cuda_stream: int) -> None:
        self.lib.check(self.lib.swlm_state_set_stream(self.state, C.c_void_p(cuda_stream)))

    def set_prefill_chunk(self, tokens: int) -> None:
        """Tokens per prompt-ingestion chunk (0: one token at a time through the decode graph)."""
        self.lib.check(self.lib.swlm_state_set_prefill_chunk(self.state, tokens))

    def prompt_snapshot(self) -> C.c_void_p:
        snap = C.c_void_p()
        self.lib.check(self.lib.swlm_state_snapshot(self.state, C.byref(snap)))
        return snap

    def restore(self, snap: C.c_void_p) -> None:
        self.lib.check(self.lib.swlm_state_restore(self.state, snap))

    def free_snapshot(self, snap: C.c_void_p) -> None:
        self.lib.swlm_snap_destroy(snap)

    def logits(self) -> np.ndarray:
        out = np.empty((self.batch, int(self.desc.vocab)), dtype=np.uint16)
        self.lib.check(self.lib.swlm_read_logits(self.state, _ptr(out), out.size))
        return out

    # -- probes -----------------------------------------------------------------------------------------
    def read_buffer(self, buf: int, count: int) -> np.ndarray:
        out = np.empty((self.batch, count), dtype=np.uint16)
        self.lib.check(self.lib.swlm_read_buffer(self.state, buf, _ptr(out), count))
        return out

    def write_buffer(self, buf: int, data_bf16: np.ndarray) -> None:
        d = np.ascontiguousarray(data_bf16, dtype=np.uint16).reshape(self.batch, -1)
        self.lib.check(self.lib.swlm_write_buffer(self.state, buf, _ptr(d), d.shape[1]))

    def read_kv(self, which: int, layer: int, b: int, head: int, count: int) -> np.ndarray:
        out = np.empty((count, int(self.desc.head_dim)), dtype=np.uint16)
        self.lib.check(self.lib.swlm_read_kv(self.state, which, layer, b, head, count, _ptr(out)))
        return out

    def write_kv(self, which: int, layer: int, b: int, head: int, rows_bf16: np.ndarray) -> None:
        d = np.ascontiguousarray(rows_bf16, dtype=np.uint16)
        self.lib.check(self.lib.swlm_write_kv(self.state, which, layer, b, head, d.shape[0], _ptr(d)))

    # rotated KV schemes: the fp16 rotors [kv_layers][kv_heads][ceil(head_dim / 3)][4] and the projected K residuals
    def rotors(self) -> np.ndarray:
        d = self.desc
        out = np.empty((int(d.kv_layers), int(d.kv_heads), (int(d.head_dim) + 2) // 3, 4), dtype=np.uint16)
        self.lib.check(self.lib.swlm_state_get_rotors(self.state, _ptr(out), out.size))
        return out

    def set_rotors(self, values_f16_bits: np.ndarray) -> None:
        v = np.ascontiguousarray(values_f16_bits, dtype=np.uint16).reshape(-1)
        self.lib.check(self.lib.swlm_state_set_rotors(self.state, _ptr(v), v.size))

    def read_qjl(self, layer: int, b: int, head: int, count: int) -> np.ndarray:
        out = np.empty((count, int(self.desc.kv_qjl_dim)), dtype=np.uint16)
        self.lib.check(self.lib.swlm_read_qjl(self.state, layer, b, head, count, _ptr(out)))
        return out

    def read_conv(self, layer: int, b: int) -> np.ndarray:
        out = np.empty((int(self.desc.conv_kernel), int(self.desc.conv_dim)), dtype=np.uint16)
        self.lib.check(self.lib.swlm_read_conv(self.state, layer, b, _ptr(out)))
        return out

    def read_ssm_state(self, layer: int, b: int) -> np.ndarray:
        d = self.desc
        out = np.empty((int(d.ssm_heads), int(d.ssm_key_dim), int(d.ssm_value_dim)), dtype=np.float32)
        self.lib.check(self.lib.swlm_read_ssm_state(self.state, layer, b, _ptr(out)))
        return out

    def set_position(self, position: int) -> None:
        self.lib.check(self.lib.swlm_set_position(self.state, position))

    # -- several sequences, each at its own position ---------------------------------------------------
    def set_positions(self, positions) -> None:
        p = np.ascontiguousarray(np.asarray(positions, dtype=np.int32).reshape(self.batch))
        self.lib.check(self.lib.swlm_set_positions(self.state, _ptr(p)))

    @property
    def positions(self) -> np.ndarray:
        out = np.empty(self.batch, dtype=np.int32)
        self.lib.check(self.lib.swlm_get_positions(self.state, _ptr(out)))
        return out

    def prefill_sequence(self, seq: int, tokens) -> int:
        """Append a prompt to one sequence only; returns that sequence's next token."""
        t = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32).reshape(-1))
        out = np.empty(1, dtype=np.int32)
        self.lib.check(self.lib.swlm_prefill_seq(self.state, seq, _ptr(t), t.size, _ptr(out)))
        return int(out[0])

    def reset_sequence(self, seq: int) -> None:
        self.lib.check(self.lib.swlm_state_reset_seq(self.state, seq))

    def run_step(self, step: Step, token_in=None) -> np.ndarray:
        tin = None
        if token_in is not None:
            t = np.ascontiguousarray(np.asarray(token_in, dtype=np.int32).reshape(self.batch))
            tin = _ptr(t)
        out = np.zeros(self.batch, dtype=np.int32)
        self.lib.check(self.lib.swlm_run_step(self.state, C.byref(step), tin, _ptr(out)))
        return out

    def profile_kind(self, step_kind: int, repeats: int) -> None:
        self.lib.check(self.lib.swlm_profile_kind(self.state, step_kind, repeats))

    @property
    def launches_per_step(self) -> int:
        return int(self.lib.swlm_plan_launch_count(self.plan))

    @property
    def launches(self) -> int:
        return int(self.lib.swlm_launches(self.state))

    def describe(self) -> str:
        need = self.lib.swlm_plan_describe(self.plan, None, 0)
        buf = C.create_string_buffer(need)
        self.lib.swlm_plan_describe(self.plan, buf, need)
        return buf.value.decode()


def load_model(store: WeightStore, builder, weights) -> InferenceModel:
    """Upload `weights` (name -> arrays, see synth.synth_model_weights) and compile the decode plan."""
    for name, kind, _shape, shard in builder.tensors():
        entry = weights[name]
        if kind == "q4":
            store.add_q4_mlx(name, entry[0], entry[1], entry[2], shard)
        elif kind == "f32":
            store.add_dense_f32(name, entry)
        else:
            store.add_dense(name, entry, shard if kind == "conv" else 0)
    return InferenceModel(store, builder.decode_steps(), builder.config.buffers_desc())


def staf_tensor_name(name: str, kind: str) -> str:
    """Name of a plan tensor inside an MLX bundle / STAF file: a quantized module `x` is stored as `x.weight` (its
    `.scales` / `.biases` companions are folded into the blocks), dense tensors keep their names."""
    return name if kind != "q4" or name.endswith(".weight") else name + ".weight"


def bundle_tensors(builder, weights):
    """The MLX-shaped safetensors tensors of a synthetic model: name -> (dtype string, array), quantized modules as
    `.weight` (u32 words) / `.scales` / `.biases` (bf16) triples."""
    out = {}
    for name, kind, _shape, _shard in builder.tensors():
        entry = weights[name]
        if kind == "q4":
            mod = staf_tensor_name(name, kind)[:-len(".weight")]
            out[mod + ".weight"] = ("U32", np.ascontiguousarray(entry[0], dtype=np.uint32))
            out[mod + ".scales"] = ("BF16", np.ascontiguousarray(entry[1], dtype=np.uint16))
            out[mod + ".biases"] = ("BF16", np.ascontiguousarray(entry[2], dtype=np.uint16))
        elif kind == "f32":
            out[name] = ("F32", np.ascontiguousarray(entry, dtype=np.float32))
        else:
            out[name] = ("BF16", np.ascontiguousarray(entry, dtype=np.uint16))
    return out


def load_model_from_staf(store: WeightStore, builder, staf_file) -> InferenceModel:
    """Upload the tensors a plan needs straight from a STAF file (4-bit group-64 / group-128 blocks as they are, dense tensors as
    bf16) and compile the decode plan. Mirrors STAFLoader.load -> STAFWeightStore
    (Sources/MetalCompiler/STAF/STAFLoader.swift:19-299) feeding MetalInferenceModel."""
    from . import staf as _staf

    for name, kind, _shape, shard in builder.tensors():
        entry = staf_file[staf_tensor_name(name, kind)]
        raw = np.asarray(staf_file.data[entry.payload_offset:entry.payload_offset + entry.payload_size])
        if kind == "q4":
            if entry.scheme not in (_staf.SCHEME_Q4_G64, _staf.SCHEME_Q4_G128):
                raise _staf.STAFError(f"{entry.name}: scheme {entry.scheme:#x} is not 4-bit group 64 or 128")
            group = 64 if entry.scheme == _staf.SCHEME_Q4_G64 else 128
            n, words = entry.shape
            store.add_q4_staf(name, raw.reshape(n, words * 8 // group, 4 + group // 2), n, words * 8, shard, group=group)
        elif kind == "f32":
            if entry.scheme != _staf.SCHEME_FP32:
                raise _staf.STAFError(f"{entry.name}: expected an fp32 section")
            store.add_dense_f32(name, raw.view(np.float32))
        else:
            if entry.scheme == _staf.SCHEME_BF16:
                arr = raw.view(np.uint16)
            elif entry.scheme == _staf.SCHEME_FP32:
                arr = _staf.f32_to_bf16(raw.view(np.float32))
            else:
                arr = _staf.f32_to_bf16(raw.view(np.float16).astype(np.float32))
            rows = int(np.prod(entry.shape[:-1])) if len(entry.shape) > 1 else 1
            store.add_dense(name, np.ascontiguousarray(arr).reshape(rows, entry.shape[-1]), shard if kind == "conv" else 0)
    return InferenceModel(store, builder.decode_steps(), builder.config.buffers_desc())
