"""ctypes binding of oracle/liboracle.so — the CPU checker. Test infrastructure only."""
import ctypes as C

import numpy as np


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


class OracleModel:
    def __init__(self, orc, desc):
        self.o = orc
        self.dll = orc.dll
        self.desc = desc
        self.batch = int(desc.max_batch)
        self.h = C.c_void_p(self.dll.orc_create(C.byref(desc)))

    def __del__(self):
        if getattr(self, "h", None):
            self.dll.orc_destroy(self.h)
            self.h = None

    def add_q4(self, name, w, s, b, staf_fp16=False):
        """The group size (64 or 128) follows from the shape of the scales."""
        w = np.ascontiguousarray(w, dtype=np.uint32); s = np.ascontiguousarray(s, dtype=np.uint16); b = np.ascontiguousarray(b, dtype=np.uint16)
        group = w.shape[1] * 8 // s.shape[1]
        rc = self.dll.orc_add_q4_group(self.h, name.encode(), w.shape[0], w.shape[1] * 8, group, _p(w), _p(s), _p(b), int(staf_fp16))
        assert rc == 0, self.error()

    def add_dense(self, name, data):
        d = np.ascontiguousarray(data, dtype=np.uint16)
        assert self.dll.orc_add_dense(self.h, name.encode(), C.c_int64(d.size), _p(d)) == 0

    def add_dense_f32(self, name, data):
        d = np.ascontiguousarray(data, dtype=np.float32)
        assert self.dll.orc_add_dense_f32(self.h, name.encode(), C.c_int64(d.size), _p(d)) == 0

    def read_ssm_state(self, layer, b):
        d = self.desc
        out = np.empty((int(d.ssm_heads), int(d.ssm_key_dim), int(d.ssm_value_dim)), dtype=np.float32)
        self.dll.orc_read_ssm_state(self.h, layer, b, _p(out))
        return out

    def load(self, builder, weights, staf_fp16=False):
        for name, kind, _shape, _shard in builder.tensors():
            if kind == "q4":
                self.add_q4(name, *weights[name], staf_fp16=staf_fp16)
            elif kind == "f32":
                self.add_dense_f32(name, weights[name])
            else:
                self.add_dense(name, weights[name])
        steps = builder.decode_steps()
        arr = (type(steps[0]) * len(steps))(*steps)
        assert self.dll.orc_set_plan(self.h, arr, len(steps)) == 0

    def error(self):
        return self.dll.orc_error(self.h).decode()

    def reset(self):
        self.dll.orc_reset(self.h)

    @property
    def position(self):
        return self.dll.orc_position(self.h)

    def set_position(self, p):
        self.dll.orc_set_position(self.h, p)

    def decode(self, token_in):
        t = np.ascontiguousarray(np.asarray(token_in, dtype=np.int32).reshape(self.batch))
        out = np.empty(self.batch, dtype=np.int32)
        rc = self.dll.orc_decode(self.h, _p(t), _p(out))
        assert rc == 0, self.error()
        return out

    def prefill(self, tokens):
        t = np.ascontiguousarray(np.atleast_2d(np.asarray(tokens, dtype=np.int32)))
        out = np.empty(self.batch, dtype=np.int32)
        rc = self.dll.orc_prefill(self.h, _p(t), t.shape[1], _p(out))
        assert rc == 0, self.error()
        return out

    def read_buffer(self, buf, count):
        out = np.empty((self.batch, count), dtype=np.uint16)
        assert self.dll.orc_read_buffer(self.h, buf, _p(out), count) == 0
        return out

    def write_buffer(self, buf, data):
        d = np.ascontiguousarray(data, dtype=np.uint16).reshape(self.batch, -1)
        assert self.dll.orc_write_buffer(self.h, buf, _p(d), d.shape[1]) == 0

    def run_step(self, step, token_in=None):
        tin = None
        if token_in is not None:
            t = np.ascontiguousarray(np.asarray(token_in, dtype=np.int32).reshape(self.batch))
            tin = _p(t)
        out = np.zeros(self.batch, dtype=np.int32)
        rc = self.dll.orc_run_step(self.h, C.byref(step), tin, _p(out))
        assert rc == 0, self.error()
        return out

    def read_kv(self, which, layer, b, head, count):
        out = np.empty((count, int(self.desc.head_dim)), dtype=np.uint16)
        self.dll.orc_read_kv(self.h, which, layer, b, head, count, _p(out))
        return out

    def write_kv(self, which, layer, b, head, rows):
        d = np.ascontiguousarray(rows, dtype=np.uint16)
        self.dll.orc_write_kv(self.h, which, layer, b, head, d.shape[0], _p(d))

    def rotors(self):
        out = np.empty(int(self.dll.orc_rotor_count(self.h)), dtype=np.uint16)
        self.dll.orc_get_rotors(self.h, _p(out))
        return out

    def set_rotors(self, values):
        d = np.ascontiguousarray(values, dtype=np.uint16).reshape(-1)
        assert d.size == int(self.dll.orc_rotor_count(self.h))
        self.dll.orc_set_rotors(self.h, _p(d))

    def qjl_matrix(self):
        out = np.empty((int(self.desc.head_dim), int(self.desc.kv_qjl_dim)), dtype=np.uint16)
        self.dll.orc_get_qjl_matrix(self.h, _p(out))
        return out

    def read_qjl(self, layer, b, head, count):
        out = np.empty((count, int(self.desc.kv_qjl_dim)), dtype=np.uint16)
        assert self.dll.orc_read_qjl(self.h, layer, b, head, count, _p(out)) == 0
        return out

    def read_conv(self, layer, b):
        out = np.empty((int(self.desc.conv_kernel), int(self.desc.conv_dim)), dtype=np.uint16)
        self.dll.orc_read_conv(self.h, layer, b, _p(out))
        return out


class Oracle:
    def __init__(self, path):
        self.dll = C.CDLL(path)
        d = self.dll
        d.orc_create.restype = C.c_void_p
        d.orc_create.argtypes = [C.c_void_p]
        d.orc_destroy.argtypes = [C.c_void_p]
        d.orc_error.restype = C.c_char_p
        d.orc_error.argtypes = [C.c_void_p]
        d.orc_add_q4.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        d.orc_add_q4_group.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        d.orc_staf_repack_mlx_group.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        d.orc_q4_dequant_staf_group.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        d.orc_add_dense.argtypes = [C.c_void_p, C.c_char_p, C.c_int64, C.c_void_p]
        d.orc_add_dense_f32.argtypes = [C.c_void_p, C.c_char_p, C.c_int64, C.c_void_p]
        d.orc_read_ssm_state.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        d.orc_set_plan.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        d.orc_reset.argtypes = [C.c_void_p]
        d.orc_position.argtypes = [C.c_void_p]
        d.orc_set_position.argtypes = [C.c_void_p, C.c_int]
        d.orc_decode.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        d.orc_prefill.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        d.orc_read_buffer.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int]
        d.orc_write_buffer.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int]
        d.orc_run_step.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        d.orc_read_kv.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
        d.orc_write_kv.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
        d.orc_read_conv.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        d.orc_rotor_count.argtypes = [C.c_void_p]
        d.orc_rotor_count.restype = C.c_int64
        d.orc_get_rotors.argtypes = [C.c_void_p, C.c_void_p]
        d.orc_set_rotors.argtypes = [C.c_void_p, C.c_void_p]
        d.orc_get_qjl_matrix.argtypes = [C.c_void_p, C.c_void_p]
        d.orc_read_qjl.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
        d.orc_q4_dequant_mlx.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        d.orc_staf_repack_mlx.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        d.orc_q4_dequant_staf.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        d.orc_q4_dequant_bf16.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        d.orc_qgemm.argtypes = [C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        d.orc_qgemm_group.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        d.orc_staf_gemv_f32.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
        d.orc_rope_bf16.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int]
        d.orc_rope_inv_freq.argtypes = [C.c_int, C.c_float, C.c_void_p]
        d.orc_set_threads.argtypes = [C.c_int]

    def set_threads(self, n):
        self.dll.orc_set_threads(n)

    def threads(self):
        return self.dll.orc_get_threads()

    def model(self, desc):
        return OracleModel(self, desc)

    def dequant_mlx(self, w, s, b):
        w = np.ascontiguousarray(w, dtype=np.uint32); s = np.ascontiguousarray(s, dtype=np.uint16); b = np.ascontiguousarray(b, dtype=np.uint16)
        n, k = w.shape[0], w.shape[1] * 8
        out = np.empty((n, k), dtype=np.float32)
        self.dll.orc_q4_dequant_mlx(n, k, _p(w), _p(s), _p(b), _p(out))
        return out

    def dequant_bf16(self, w, s, b):
        w = np.ascontiguousarray(w, dtype=np.uint32); s = np.ascontiguousarray(s, dtype=np.uint16); b = np.ascontiguousarray(b, dtype=np.uint16)
        n, k = w.shape[0], w.shape[1] * 8
        out = np.empty((n, k), dtype=np.uint16)
        self.dll.orc_q4_dequant_bf16(n, k, _p(w), _p(s), _p(b), _p(out))
        return out

    def staf_repack(self, w, s, b):
        w = np.ascontiguousarray(w, dtype=np.uint32); s = np.ascontiguousarray(s, dtype=np.uint16); b = np.ascontiguousarray(b, dtype=np.uint16)
        n, k = w.shape[0], w.shape[1] * 8
        out = np.empty((n, k // 64, 36), dtype=np.uint8)
        self.dll.orc_staf_repack_mlx(n, k, _p(w), _p(s), _p(b), _p(out))
        return out

    def staf_repack_group(self, w, s, b, group):
        w = np.ascontiguousarray(w, dtype=np.uint32); s = np.ascontiguousarray(s, dtype=np.uint16); b = np.ascontiguousarray(b, dtype=np.uint16)
        n, k = w.shape[0], w.shape[1] * 8
        out = np.empty((n, k // group, 4 + group // 2), dtype=np.uint8)
        self.dll.orc_staf_repack_mlx_group(n, k, group, _p(w), _p(s), _p(b), _p(out))
        return out

    def dequant_staf_group(self, blocks, n, k, group):
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        out = np.empty((n, k), dtype=np.float32)
        self.dll.orc_q4_dequant_staf_group(n, k, group, _p(blocks), _p(out))
        return out

    def dequant_staf(self, blocks, n, k):
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        out = np.empty((n, k), dtype=np.float32)
        self.dll.orc_q4_dequant_staf(n, k, _p(blocks), _p(out))
        return out

    def staf_gemv_f32(self, blocks, n, k, x):
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8); x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty(n, dtype=np.float32)
        self.dll.orc_staf_gemv_f32(n, k, _p(blocks), _p(x), _p(y))
        return y

    def qgemm(self, x_bf16, w, s, b, staf_fp16=False, want_f64=False):
        x = np.ascontiguousarray(x_bf16, dtype=np.uint16)
        w = np.ascontiguousarray(w, dtype=np.uint32); s = np.ascontiguousarray(s, dtype=np.uint16); b = np.ascontiguousarray(b, dtype=np.uint16)
        m, k = x.shape
        n = w.shape[0]
        y = np.empty((m, n), dtype=np.uint16)
        y64 = np.empty((m, n), dtype=np.float64) if want_f64 else None
        rc = self.dll.orc_qgemm_group(m, n, k, k // s.shape[1], _p(x), _p(w), _p(s), _p(b), _p(y), _p(y64) if want_f64 else None, int(staf_fp16))
        assert rc == 0
        return (y, y64) if want_f64 else y

    def rope_bf16(self, v_bf16, heads, head_dim, rope_dim, base, position):
        v = np.array(v_bf16, dtype=np.uint16, copy=True)
        self.dll.orc_rope_bf16(_p(v), heads, head_dim, rope_dim, C.c_float(base), position)
        return v
