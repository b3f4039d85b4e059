"""NeoML CDnn graphs on the hosted libraries (neoml_b200/lib/host): ctypes mirror of host/cdnn_host.cpp.

The libraries are NeoML itself (libNeoML.so, built unmodified from a NeoML checkout) on a libNeoMathEngine.so whose
GPU factory returns the B200 engine.  `Engine("gpu")` is NeoML's CreateGpuMathEngine, `Engine("cpu")` its own CPU
engine; a `Net` is a CDnn loaded from a `Model` archive on one of them.

Load this module in a process that has not loaded another libNeoMathEngine.so: both carry the same soname.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

HOST_DIR = Path(__file__).resolve().parent / "lib" / "host"
_dir = HOST_DIR
_lib = None

_fp = C.POINTER(C.c_float)
_ip = C.POINTER(C.c_int)


def available() -> bool:
    return (_dir / "libcdnn_host.so").exists()


def use_directory(path) -> None:
    """Before the first load(): take libcdnn_host.so (and the NeoML / NeoMathEngine libraries beside it) from `path`
    instead of neoml_b200/lib/host -- e.g. a build of the same harness on an unmodified NeoMathEngine."""
    global _dir
    if _lib is not None:
        raise RuntimeError("the libraries are loaded already")
    _dir = Path(path)


def directory() -> Path:
    return _dir


def load():
    global _lib
    if _lib is not None:
        return _lib
    path = _dir / "libcdnn_host.so"
    if not path.exists():
        raise RuntimeError(f"{path} is missing: run `make -C neoml_b200/host` where a NeoML checkout is available")
    lib = C.CDLL(str(path), mode=C.RTLD_GLOBAL)
    lib.cdnn_last_error.restype = C.c_char_p
    lib.cdnn_engine_create.restype = C.c_void_p
    lib.cdnn_engine_create.argtypes = [C.c_int, C.c_int, C.c_ulonglong, C.c_int]
    lib.cdnn_engine_destroy.argtypes = [C.c_void_p]
    lib.cdnn_engine_info.argtypes = [C.c_void_p, _ip, C.c_char_p, C.c_int, C.POINTER(C.c_ulonglong)]
    lib.cdnn_gpu_count.restype = C.c_int
    lib.cdnn_model_destroy.argtypes = [C.c_void_p]
    lib.cdnn_model_bytes.restype = C.c_longlong
    lib.cdnn_model_bytes.argtypes = [C.c_void_p]
    lib.cdnn_model_conv.restype = C.c_void_p
    lib.cdnn_model_conv.argtypes = [_ip, _fp, _fp]
    lib.cdnn_model_mbv2.restype = C.c_void_p
    lib.cdnn_model_mbv2.argtypes = [C.c_int] * 5 + [C.c_float] * 2 + [_fp] * 6
    lib.cdnn_model_matmul.restype = C.c_void_p
    lib.cdnn_model_resnet50.restype = C.c_void_p
    lib.cdnn_model_resnet50.argtypes = [_fp, C.c_longlong, C.c_int]
    lib.cdnn_model_transformer.restype = C.c_void_p
    lib.cdnn_model_transformer.argtypes = [C.c_int] * 4 + [C.c_ulonglong, C.c_float, C.c_int]
    lib.cdnn_net_create.restype = C.c_void_p
    lib.cdnn_net_create.argtypes = [C.c_void_p, C.c_void_p]
    lib.cdnn_net_destroy.argtypes = [C.c_void_p]
    lib.cdnn_net_set_input.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, _ip]
    lib.cdnn_net_run.argtypes = [C.c_void_p]
    lib.cdnn_net_get_output.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_longlong, _ip, _ip]
    lib.cdnn_net_time_steps.restype = C.c_double
    lib.cdnn_net_time_steps.argtypes = [C.c_void_p, C.c_int, C.c_char_p, C.c_void_p, C.c_char_p, C.c_void_p, C.c_longlong]
    lib.cdnn_net_time_steps_double_buffered.restype = C.c_double
    lib.cdnn_net_time_steps_double_buffered.argtypes = [C.c_void_p, C.c_int, C.c_char_p, C.c_void_p, C.c_longlong, C.c_char_p,
                                                        C.c_void_p, C.c_longlong, C.c_longlong]
    lib.cdnn_replicas_create.restype = C.c_void_p
    lib.cdnn_replicas_create.argtypes = [C.c_int, C.c_int, _ip, C.c_void_p]
    lib.cdnn_replicas_destroy.argtypes = [C.c_void_p]
    lib.cdnn_replicas_net.restype = C.c_void_p
    lib.cdnn_replicas_net.argtypes = [C.c_void_p, C.c_int]
    for fn in (lib.cdnn_replicas_time_steps, lib.cdnn_replicas_time_steps_double_buffered):
        fn.restype = C.c_double
        fn.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_char_p, C.c_void_p, C.c_longlong,
                       C.c_char_p, C.c_void_p, C.c_longlong]
    if hasattr(lib, "cdnn_selftest_free_while_pending"):
        lib.cdnn_selftest_free_while_pending.argtypes = [C.c_void_p, _fp]
        lib.cdnn_selftest_abort_distributed.argtypes = [_ip, C.c_char_p, C.c_int]
    if hasattr(lib, "cdnn_selftest_padded_pool"):
        lib.cdnn_selftest_padded_pool.argtypes = [C.c_void_p, _ip, _ip]
    if hasattr(lib, "cdnn_selftest_random_program"):
        lib.cdnn_selftest_random_program.argtypes = [C.c_void_p, C.c_ulonglong, C.c_int, _fp, C.c_int]
    if hasattr(lib, "cdnn_selftest_product_chain"):
        lib.cdnn_selftest_product_chain.argtypes = [C.c_void_p, _fp]
    if hasattr(lib, "cdnn_selftest_normalization_chain"):
        lib.cdnn_selftest_normalization_chain.argtypes = [C.c_void_p, _fp, _ip]
    if hasattr(lib, "cdnn_selftest_attention_chain"):
        lib.cdnn_selftest_attention_chain.argtypes = [C.c_void_p, _fp, _ip]
    _lib = lib
    return lib


class CDnnError(RuntimeError):
    pass


def _fail(what: str):
    raise CDnnError(f"{what}: {load().cdnn_last_error().decode(errors='replace')}")


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(_fp)


class Engine:
    """kind: "cpu" (CreateCpuMathEngine), "gpu" (CreateGpuMathEngine) or "manager" (entry `device` of
    CreateGpuMathEngineManager).  flags: the reference's GPU engine flags (TF32 opt-in = 1 << 1)."""

    def __init__(self, kind: str = "gpu", device: int = 0, memory_limit: int = 0, flags: int = 0):
        self.kind = kind
        self.ptr = load().cdnn_engine_create({"cpu": 0, "gpu": 1, "manager": 2}[kind], device, memory_limit, flags)
        if not self.ptr:
            _fail(f"creating the {kind} math engine")

    def info(self):
        t, peak, name = C.c_int(), C.c_ulonglong(), C.create_string_buffer(256)
        if load().cdnn_engine_info(self.ptr, C.byref(t), name, 256, C.byref(peak)) != 0:
            _fail("engine info")
        return {"type": t.value, "name": name.value.decode(), "peak_bytes": peak.value}

    def close(self):
        if self.ptr:
            load().cdnn_engine_destroy(self.ptr)
            self.ptr = None


class Model:
    def __init__(self, ptr, what: str):
        if not ptr:
            _fail(f"building the {what} model")
        self.ptr = ptr

    @property
    def nbytes(self) -> int:
        return load().cdnn_model_bytes(self.ptr)

    def close(self):
        if self.ptr:
            load().cdnn_model_destroy(self.ptr)
            self.ptr = None

    @staticmethod
    def conv(filt, bias, stride=(1, 1), padding=(0, 0), dilation=(1, 1)):
        filt = _f32(filt)
        k, r, s, c = filt.shape
        g = (C.c_int * 10)(c, k, r, s, stride[0], stride[1], padding[0], padding[1], dilation[0], dilation[1])
        bias = _f32(bias)
        return Model(load().cdnn_model_conv(g, _ptr(filt), _ptr(bias)), "convolution")

    @staticmethod
    def mbv2(we, be, wd, bd, wp, bp, stride=1, residual=True, act1=6.0, act2=6.0):
        we, be, wd, bd, wp, bp = map(_f32, (we, be, wd, bd, wp, bp))
        cexp, cin = we.shape[0], we.shape[-1]
        cout = wp.shape[0]
        return Model(load().cdnn_model_mbv2(cin, cexp, cout, stride, int(residual), act1, act2, _ptr(we), _ptr(be),
                                            _ptr(wd), _ptr(bd), _ptr(wp), _ptr(bp)), "MobileNetV2 block")

    @staticmethod
    def matmul():
        return Model(load().cdnn_model_matmul(), "matrix multiplication")

    @staticmethod
    def resnet50(weights: dict, classes: int = 1000):
        """weights: the dictionary of neoml_b200.resnet50.make_weights()."""
        from .resnet50 import conv_specs
        order = []
        specs = {sp.name: sp for sp in conv_specs()}
        names = ["stem"]
        for sp in conv_specs():
            if sp.name.endswith("_c1"):
                p = sp.name[:-3]
                if p + "_down" in specs:
                    names.append(p + "_down")
                names += [p + "_c1", p + "_c2", p + "_c3"]
        for n in names:
            order += [weights[n + ".w"].ravel(), weights[n + ".b"].ravel()]
        order += [weights["fc.w"].ravel(), weights["fc.b"].ravel()]
        flat = np.ascontiguousarray(np.concatenate(order), dtype=np.float32)
        return Model(load().cdnn_model_resnet50(_ptr(flat), flat.size, classes), "ResNet-50")

    @staticmethod
    def transformer(layers=12, hidden=768, heads=12, ffn=3072, seed=7, sigma=0.02, mask=True):
        return Model(load().cdnn_model_transformer(layers, hidden, heads, ffn, seed, sigma, int(mask)), "transformer")


class Net:
    def __init__(self, engine: Engine, model: Model, _ptr_=None):
        self.engine = engine
        self.owned = _ptr_ is None
        self.ptr = _ptr_ or load().cdnn_net_create(engine.ptr, model.ptr)
        if not self.ptr:
            _fail("loading the model into a CDnn")

    def set_input(self, name: str, array, dims7=None):
        """array: float32 numpy array (or anything with a ctypes-able .ctypes / data pointer given as int).
        dims7 defaults to NeoML's image layout for 4-D arrays [batch, h, w, c] and sequence layout for 3-D
        [batch, seq, channels]."""
        a = _f32(array)
        if dims7 is None:
            if a.ndim == 4:
                dims7 = (1, a.shape[0], 1, a.shape[1], a.shape[2], 1, a.shape[3])
            elif a.ndim == 3:
                dims7 = (1, a.shape[0], a.shape[1], 1, 1, 1, a.shape[2])
            elif a.ndim == 2:
                dims7 = (1, a.shape[0], 1, 1, 1, 1, a.shape[1])
            else:
                raise ValueError("give dims7 for this array")
        d = (C.c_int * 7)(*dims7)
        if load().cdnn_net_set_input(self.ptr, name.encode(), a.ctypes.data_as(C.c_void_p), d) != 0:
            _fail(f"set_input({name})")

    def set_input_ptr(self, name: str, host_ptr: int, dims7):
        d = (C.c_int * 7)(*dims7)
        if load().cdnn_net_set_input(self.ptr, name.encode(), C.c_void_p(host_ptr), d) != 0:
            _fail(f"set_input({name})")

    def run(self):
        if load().cdnn_net_run(self.ptr) != 0:
            _fail("RunOnce")

    def output(self, name: str):
        d, is_int = (C.c_int * 7)(), C.c_int()
        if load().cdnn_net_get_output(self.ptr, name.encode(), None, 0, d, C.byref(is_int)) != 0:
            _fail(f"output({name})")
        out = np.empty(tuple(d), dtype=np.int32 if is_int.value else np.float32)
        if load().cdnn_net_get_output(self.ptr, name.encode(), out.ctypes.data_as(C.c_void_p), out.nbytes, d,
                                      C.byref(is_int)) != 0:
            _fail(f"output({name})")
        return out

    def time_steps(self, steps: int, sink: str, source: str | None = None, input_ptr: int | None = None,
                   output_ptr: int | None = None, output_bytes: int = 0, double_buffered: bool = False,
                   input_stride_floats: int = 0, output_stride_bytes: int = 0) -> float:
        """Wall-clock seconds of `steps` x (host -> source blob, RunOnce, sinks -> host).  double_buffered: the input
        copy of step i+1 is issued before the results of step i are read (see host/cdnn_host.cpp); the strides let
        every step have its own batch and result buffer."""
        if double_buffered:
            t = load().cdnn_net_time_steps_double_buffered(
                self.ptr, steps, source.encode() if source else None, C.c_void_p(input_ptr) if input_ptr else None,
                input_stride_floats, sink.encode(), C.c_void_p(output_ptr) if output_ptr else None, output_stride_bytes,
                output_bytes)
            if t < 0:
                _fail("time_steps")
            return t
        t = load().cdnn_net_time_steps(self.ptr, steps, source.encode() if source else None,
                                       C.c_void_p(input_ptr) if input_ptr else None, sink.encode(),
                                       C.c_void_p(output_ptr) if output_ptr else None, output_bytes)
        if t < 0:
            _fail("time_steps")
        return t

    def close(self):
        if self.ptr and self.owned:
            load().cdnn_net_destroy(self.ptr)
        self.ptr = None


def selftest_free_while_pending(engine: Engine) -> float:
    """See cdnn_selftest_free_while_pending in host/cdnn_host.cpp: largest difference between a convolution + ReLU
    whose source blob was freed right after the convolution call and the same with the source kept alive."""
    worst = C.c_float(-1.0)
    if load().cdnn_selftest_free_while_pending(engine.ptr, C.byref(worst)) != 0:
        _fail("selftest_free_while_pending")
    return worst.value


def selftest_padded_pool(engine: Engine) -> tuple[int, int]:
    """See cdnn_selftest_padded_pool: (values that differ from the host evaluation, kernels launched by pad + pool)."""
    wrong, launches = C.c_int(-1), C.c_int(-1)
    if load().cdnn_selftest_padded_pool(engine.ptr, C.byref(wrong), C.byref(launches)) != 0:
        _fail("selftest_padded_pool")
    return wrong.value, launches.value


def selftest_attention_chain(engine: Engine) -> tuple[float, int]:
    """See cdnn_selftest_attention_chain: (largest error relative to the RMS of the expected values, kernels launched by
    the five calls of the chain)."""
    worst, launches = C.c_float(-1), C.c_int(-1)
    if load().cdnn_selftest_attention_chain(engine.ptr, C.byref(worst), C.byref(launches)) != 0:
        _fail("selftest_attention_chain")
    return worst.value, launches.value


RANDOM_PROGRAM_STATE_FLOATS = 6 * 24 * 32 + 4 * 24 + 3 * 32 + 2


def selftest_random_program(engine: Engine, seed: int, steps: int):
    """See cdnn_selftest_random_program: the final contents of all its buffers after `steps` random calls."""
    state = np.zeros(RANDOM_PROGRAM_STATE_FLOATS, np.float32)
    if load().cdnn_selftest_random_program(engine.ptr, seed, steps, state.ctypes.data_as(_fp), state.size) != 0:
        _fail("selftest_random_program")
    return state


def selftest_product_chain(engine: Engine) -> float:
    """See cdnn_selftest_product_chain: the largest error relative to the RMS of the expected values."""
    worst = C.c_float(-1)
    if load().cdnn_selftest_product_chain(engine.ptr, C.byref(worst)) != 0:
        _fail("selftest_product_chain")
    return worst.value


def selftest_normalization_chain(engine: Engine) -> tuple[float, int]:
    """See cdnn_selftest_normalization_chain: (largest relative difference from the host evaluation, kernels launched by
    the output chain and its read)."""
    worst, launches = C.c_float(-1), C.c_int(-1)
    if load().cdnn_selftest_normalization_chain(engine.ptr, C.byref(worst), C.byref(launches)) != 0:
        _fail("selftest_normalization_chain")
    return worst.value, launches.value


def selftest_abort_distributed(devices=(0, 1)) -> str:
    """See cdnn_selftest_abort_distributed: returns the message of the AllReduce that followed a peer's abort."""
    d = (C.c_int * 2)(*devices)
    message = C.create_string_buffer(1024)
    if load().cdnn_selftest_abort_distributed(d, message, len(message)) != 0:
        _fail("selftest_abort_distributed")
    return message.value.decode(errors="replace")


class Replicas:
    """`count` replicas of one model, one engine and host thread each.  kind "cpu": CreateCpuMathEngine each;
    kind "gpu": NeoML's CreateDistributedCudaMathEngines on `devices`."""

    def __init__(self, kind: str, model: Model, count: int | None = None, devices=None):
        devices = list(devices) if devices is not None else list(range(count or 1))
        self.count = count if count is not None else len(devices)
        d = (C.c_int * max(1, len(devices)))(*devices)
        self.ptr = load().cdnn_replicas_create(0 if kind == "cpu" else 1, self.count, d, model.ptr)
        if not self.ptr:
            _fail("creating the replicas")

    def net(self, i: int) -> Net:
        return Net(None, None, _ptr_=load().cdnn_replicas_net(self.ptr, i))

    def time_steps(self, warmup: int, steps: int, source: str, inputs_ptr: int, input_floats_per_replica: int,
                   sink: str, outputs_ptr: int, output_bytes_per_replica: int, double_buffered: bool = False) -> float:
        """Seconds until the last replica finished `steps` x (host -> source blob, RunOnce, sink -> host), all replicas
        started together on one thread each.  double_buffered: every replica issues the input copy of step i+1
        before it reads the results of step i."""
        fn = load().cdnn_replicas_time_steps_double_buffered if double_buffered else load().cdnn_replicas_time_steps
        t = fn(self.ptr, warmup, steps, source.encode(),
               C.c_void_p(inputs_ptr) if inputs_ptr else None, input_floats_per_replica,
               sink.encode(), C.c_void_p(outputs_ptr) if outputs_ptr else None,
               output_bytes_per_replica)
        if t < 0:
            _fail("replicas time_steps")
        return t

    def close(self):
        if self.ptr:
            load().cdnn_replicas_destroy(self.ptr)
            self.ptr = None
