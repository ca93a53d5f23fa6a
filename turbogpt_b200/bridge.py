"""ctypes interface to libturbogpt_b200.so, mirroring the reference's tests/bridge.py:7-81
(same class names, fields, defaults and methods) and adding the extended configuration.

The library path can be overridden with TURBOGPT_LIBRARY, as in the reference bridge
(tests/bridge.py:32-33).  Loading fails loudly when the library has not been built.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

_PACKAGE = Path(__file__).resolve().parent

NORM_RMS, NORM_LAYER = 0, 1
ATTENTION_ARGMAX, ATTENTION_SOFTMAX = 0, 1
MLP_SWIGLU, MLP_GELU = 0, 1
ROPE_NONE, ROPE_PARTIAL = 0, 1
HIDDEN_MUON, HIDDEN_ADAMW = 0, 1
PRECISION_BF16, PRECISION_FP32 = 0, 1
FLAG_NO_TENSOR_CORES, FLAG_PROFILE, FLAG_BF16_GRADIENT_EXCHANGE, FLAG_NO_GRAPH, FLAG_NO_COMMUNICATOR = 1, 2, 4, 8, 16


class Config(C.Structure):
    """config.h:5-13 (72 bytes)."""
    _fields_ = [(x, C.c_int) for x in ('depth', 'context', 'batch', 'device', 'blocks', 'ns_steps')] + [
        (x, C.c_float) for x in ('learning_rate', 'muon_lr', 'beta1', 'beta2', 'momentum',
                                 'weight_decay', 'epsilon', 'clip')] + [('seed', C.c_uint64), ('inflight', C.c_int)]

    def __init__(self, **kwargs):
        super().__init__(4, 4, 16, 0, 0, 5, .0006, .02, .9, .95, .95, .1, 1e-8, 1., 3407, 1)
        for key, value in kwargs.items():
            setattr(self, key, value)


class ConfigEx(C.Structure):
    """TgConfigEx of include/turbogpt_b200.h."""
    _fields_ = [('base', Config), ('struct_size', C.c_int32)] + [
        (x, C.c_int32) for x in ('width', 'heads', 'hidden', 'norm', 'attention', 'mlp', 'tied', 'rope',
                                 'hidden_optimizer', 'precision', 'world', 'rank', 'flags')] + [
        ('nccl_id', C.c_uint8 * 128)]

    @classmethod
    def reference(cls, base: Config | None = None, **kwargs) -> "ConfigEx":
        c = cls()
        load_library().tg_ex_reference_config(C.byref(base or Config()), C.byref(c))
        for key, value in kwargs.items():
            setattr(c, key, value)
        return c

    @classmethod
    def gpt(cls, base: Config, width: int, heads: int, hidden: int | None = None, **kwargs) -> "ConfigEx":
        c = cls()
        load_library().tg_ex_gpt_config(C.byref(base), width, heads, hidden or 4 * width, C.byref(c))
        for key, value in kwargs.items():
            setattr(c, key, value)
        return c


class OneCycle(C.Structure):
    """optim.h:6-13."""
    _fields_ = [('total_steps', C.c_int)] + [
        (name, C.c_double) for name in ('warmup_fraction', 'initial_lr_fraction',
                                        'final_lr_fraction', 'low_momentum', 'high_momentum')]

    def __init__(self, total_steps=0):
        super().__init__(total_steps, .3, .04, .000004, .85, .95)


class Checkpoint(C.Structure):
    """TgCheckpoint of include/turbogpt_b200.h: training state with caller-owned arrays."""
    _fields_ = [('weights', C.c_void_p), ('momentum', C.c_void_p), ('variance', C.c_void_p),
                ('final_loss_sums', C.c_void_p), ('step', C.c_uint64), ('final_loss_batches', C.c_uint64),
                ('train_seconds', C.c_double), ('scheduler', OneCycle)]


class StepRates(C.Structure):
    """optim.h:14-16."""
    _fields_ = [('multiplier', C.c_float), ('momentum', C.c_float)]


def library_path() -> Path:
    return Path(os.environ.get('TURBOGPT_LIBRARY', str(_PACKAGE / 'libturbogpt_b200.so')))


_library = None


def declare_reference_interface(lib: C.CDLL) -> C.CDLL:
    """ctypes signatures of the 22 functions of the reference's runtime.h on any library that
    exports them (this one, or the reference's own engine)."""
    P, I, I64 = C.c_void_p, C.c_int, C.c_int64
    lib.tg_error.restype = C.c_char_p
    lib.tg_create.argtypes = [C.POINTER(Config)]
    lib.tg_create.restype = P
    lib.tg_destroy.restype = None
    for name in ('destroy', 'parameter_count', 'blocks', 'shared_bytes', 'synchronize'):
        getattr(lib, 'tg_' + name).argtypes = [P]
    for name in ('set_weights', 'get_weights'):
        getattr(lib, 'tg_' + name).argtypes = [P, P]
    lib.tg_get_optimizer_state.argtypes = [P, P, P, C.POINTER(C.c_uint64)]
    lib.tg_set_optimizer_state.argtypes = [P, P, P, C.c_uint64]
    lib.tg_memory.argtypes = [P, C.POINTER(C.c_double)]
    lib.tg_set_data.argtypes = [P, P, I64]
    lib.tg_train.argtypes = [P, I]
    lib.tg_get_training_losses.argtypes = [P, P, I]
    lib.tg_training_versions.argtypes = [P, P, I]
    lib.tg_pipeline_stats.argtypes = [P, C.POINTER(C.c_double), C.POINTER(C.c_int)]
    lib.tg_batch.argtypes = [P] * 6
    lib.tg_predict.argtypes = [P, P, P]
    lib.tg_optimizer_test.argtypes = [P, P, I]
    lib.tg_set_onecycle.argtypes = [P, C.POINTER(OneCycle)]
    lib.tg_onecycle_point.argtypes = [C.POINTER(OneCycle), I, C.POINTER(StepRates)]
    return lib


def load_library() -> C.CDLL:
    """Loads the CUDA library and declares every export.  Raises if it is missing: there is
    no fallback implementation."""
    global _library
    if _library is not None:
        return _library
    path = library_path()
    if not path.exists():
        raise RuntimeError(f"{path} is not built; run `python -m turbogpt_b200.build` (needs nvcc)")
    lib = C.CDLL(str(path))
    P, I, I64 = C.c_void_p, C.c_int, C.c_int64
    lib.tg_error.restype = C.c_char_p
    lib.tg_create.argtypes = [C.POINTER(Config)]
    lib.tg_create.restype = P
    lib.tg_create_ex.argtypes = [C.POINTER(ConfigEx)]
    lib.tg_create_ex.restype = P
    lib.tg_destroy.restype = None
    for name in ('destroy', 'parameter_count', 'blocks', 'shared_bytes', 'synchronize'):
        getattr(lib, 'tg_' + name).argtypes = [P]
    for name in ('set_weights', 'get_weights'):
        getattr(lib, 'tg_' + name).argtypes = [P, P]
    lib.tg_get_optimizer_state.argtypes = [P, P, P, C.POINTER(C.c_uint64)]
    lib.tg_set_optimizer_state.argtypes = [P, P, P, C.c_uint64]
    lib.tg_memory.argtypes = [P, C.POINTER(C.c_double)]
    lib.tg_set_data.argtypes = [P, P, I64]
    lib.tg_train.argtypes = [P, I]
    lib.tg_get_training_losses.argtypes = [P, P, I]
    lib.tg_training_versions.argtypes = [P, P, I]
    lib.tg_pipeline_stats.argtypes = [P, C.POINTER(C.c_double), C.POINTER(C.c_int)]
    lib.tg_batch.argtypes = [P] * 6
    lib.tg_predict.argtypes = [P, P, P]
    lib.tg_optimizer_test.argtypes = [P, P, I]
    lib.tg_set_onecycle.argtypes = [P, C.POINTER(OneCycle)]
    lib.tg_onecycle_point.argtypes = [C.POINTER(OneCycle), I, C.POINTER(StepRates)]
    lib.tg_ex_reference_config.argtypes = [C.POINTER(Config), C.POINTER(ConfigEx)]
    lib.tg_ex_reference_config.restype = None
    lib.tg_ex_gpt_config.argtypes = [C.POINTER(Config), I, I, I, C.POINTER(ConfigEx)]
    lib.tg_ex_gpt_config.restype = None
    lib.tg_ex_parameter_count.argtypes = [C.POINTER(ConfigEx)]
    lib.tg_ex_parameter_count.restype = I64
    lib.tg_ex_parameter_layout.argtypes = [C.POINTER(ConfigEx), P, P, P, I]
    lib.tg_ex_initialize_weights.argtypes = [C.POINTER(ConfigEx), P]
    lib.tg_ex_save_checkpoint.argtypes = [C.c_char_p, C.POINTER(ConfigEx), C.POINTER(Checkpoint)]
    lib.tg_ex_load_checkpoint.argtypes = [C.c_char_p, C.POINTER(ConfigEx), C.POINTER(Checkpoint)]
    lib.tg_ex_config_digest.argtypes = [C.POINTER(ConfigEx)]
    lib.tg_ex_config_digest.restype = C.c_uint64
    lib.tg_ex_nccl_unique_id.argtypes = [P]
    lib.tg_ex_stream.argtypes = [P]
    lib.tg_ex_stream.restype = P
    lib.tg_ex_sample.argtypes = [P, C.c_uint64, P, P]
    lib.tg_ex_train_mean_loss.argtypes = [P, I, C.POINTER(C.c_float)]
    lib.tg_ex_train_batch.argtypes = [P, P, P, P]
    lib.tg_ex_profile.argtypes = [P, P, P, P, I, I]
    lib.tg_ex_selftest_bounded_wait.argtypes = [P, C.c_double]
    lib.tg_ex_launch_count.argtypes = [P]
    lib.tg_ex_launch_count.restype = I64
    lib.tg_ex_read_activation.argtypes = [P, I, C.c_char_p, P, I64]
    lib.tg_ex_read_activation.restype = I64
    lib.tg_ex_gemm.argtypes = [P, I64, I64, P, I64, I64, P, I64, I, I, I, I, I, P]
    lib.tg_ex_weight_gradient_static.argtypes = [P, P, P, I, I, I, P]
    lib.tg_ex_last_device_error.argtypes = [P]
    lib.tg_ex_attention_forward.argtypes = [P, P, P, I, I, I, I, I, P]
    lib.tg_ex_attention_backward.argtypes = [P, P, P, P, P, I, I, I, I, I, P]
    lib.tg_ex_norm_forward.argtypes = [I, P, P, P, P, P, P, P, I, I, P]
    lib.tg_ex_norm_backward.argtypes = [I, P, P, P, P, P, P, P, P, P, I, I, P]
    lib.tg_ex_cross_entropy.argtypes = [P, P, P, P, I, C.c_float, P]
    lib.tg_ex_head_cross_entropy.argtypes = [P, P, P, P, P, I, I, C.c_float, P]
    _library = lib
    return lib


EXPORTS = ('error create destroy parameter_count blocks shared_bytes set_weights get_weights get_optimizer_state '
           'set_optimizer_state memory set_data train get_training_losses training_versions pipeline_stats '
           'onecycle_point set_onecycle batch predict optimizer_test synchronize').split()
EXTENSIONS = ('reference_config gpt_config parameter_count parameter_layout initialize_weights config_digest save_checkpoint load_checkpoint nccl_unique_id '
              'stream sample train_mean_loss train_batch profile launch_count read_activation selftest_bounded_wait gemm weight_gradient_static last_device_error attention_forward attention_backward '
              'norm_forward norm_backward cross_entropy head_cross_entropy').split()


class Native:
    """An engine.  ``Native(Config(...))`` is the reference architecture exactly as
    tests/bridge.py's Native; ``Native(ConfigEx...)`` any architecture."""

    def __init__(self, config, library=None):
        self.lib = lib = library or load_library()
        if isinstance(config, ConfigEx):
            self.extended, self.config = config, config.base
            self.handle = lib.tg_create_ex(C.byref(config))
        else:
            self.extended, self.config = None, config
            self.handle = lib.tg_create(C.byref(config))
        if not self.handle:
            raise RuntimeError(lib.tg_error().decode())
        self.count = lib.tg_parameter_count(self.handle)

    def check(self, value):
        if value < 0:
            raise RuntimeError(self.lib.tg_error().decode())
        return value

    def close(self):
        if self.handle:
            self.lib.tg_destroy(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def set_weights(self, w):
        w = np.ascontiguousarray(w, dtype=np.float32)
        assert w.size == self.count
        self.check(self.lib.tg_set_weights(self.handle, w.ctypes.data))

    def weights(self):
        w = np.empty(self.count, np.float32)
        self.check(self.lib.tg_get_weights(self.handle, w.ctypes.data))
        return w

    def batch(self, x, y, backward=True):
        x, y = np.ascontiguousarray(x, dtype=np.uint8), np.ascontiguousarray(y, dtype=np.uint8)
        assert x.shape == y.shape == (self.config.batch, self.config.context)
        logits = np.empty((*x.shape, 256), np.float32)
        grad = np.empty(self.count, np.float32) if backward else None
        losses = np.empty(self.config.context, np.float32)
        self.check(self.lib.tg_batch(self.handle, x.ctypes.data, y.ctypes.data, logits.ctypes.data,
                                     grad.ctypes.data if grad is not None else None, losses.ctypes.data))
        return logits, grad, losses

    # ---- beyond the reference bridge ----
    def set_data(self, data):
        data = np.ascontiguousarray(data, dtype=np.uint8)
        self.check(self.lib.tg_set_data(self.handle, data.ctypes.data, len(data)))

    def set_onecycle(self, total_steps):
        self.check(self.lib.tg_set_onecycle(self.handle, C.byref(OneCycle(total_steps))))

    def train(self, steps):
        self.check(self.lib.tg_train(self.handle, steps))

    def training_losses(self, count):
        out = np.empty((count, self.config.context), np.float32)
        self.check(self.lib.tg_get_training_losses(self.handle, out.ctypes.data, count))
        return out

    def train_batch(self, x, y, want_losses=True):
        x, y = np.ascontiguousarray(x, dtype=np.uint8), np.ascontiguousarray(y, dtype=np.uint8)
        out = np.empty(self.config.context, np.float32) if want_losses else None
        self.check(self.lib.tg_ex_train_batch(self.handle, x.ctypes.data, y.ctypes.data,
                                              out.ctypes.data if want_losses else None))
        return out

    def optimizer_test(self, gradient, steps=1):
        g = np.ascontiguousarray(gradient, dtype=np.float32)
        assert g.size == self.count
        self.check(self.lib.tg_optimizer_test(self.handle, g.ctypes.data, steps))

    def optimizer_state(self):
        m, v = np.empty(self.count, np.float32), np.empty(self.count, np.float32)
        step = C.c_uint64()
        self.check(self.lib.tg_get_optimizer_state(self.handle, m.ctypes.data, v.ctypes.data, C.byref(step)))
        return m, v, step.value

    def set_optimizer_state(self, m, v, step):
        m, v = np.ascontiguousarray(m, dtype=np.float32), np.ascontiguousarray(v, dtype=np.float32)
        self.check(self.lib.tg_set_optimizer_state(self.handle, m.ctypes.data, v.ctypes.data, step))

    def predict(self, context):
        context = np.ascontiguousarray(context, dtype=np.uint8)
        assert context.size == self.config.context
        logits = np.empty(256, np.float32)
        self.check(self.lib.tg_predict(self.handle, context.ctypes.data, logits.ctypes.data))
        return logits

    def sample(self, step):
        x = np.empty((self.config.batch, self.config.context), np.uint8)
        y = np.empty_like(x)
        self.check(self.lib.tg_ex_sample(self.handle, step, x.ctypes.data, y.ctypes.data))
        return x, y

    def activation(self, layer, name):
        """An activation of the last forward pass as FP32 [tokens, features] (diagnostic)."""
        count = self.lib.tg_ex_read_activation(self.handle, layer, name.encode(), None, 0)
        if count < 0:
            raise RuntimeError(self.lib.tg_error().decode())
        out = np.empty(count, np.float32)
        self.check(self.lib.tg_ex_read_activation(self.handle, layer, name.encode(), out.ctypes.data, count))
        return out.reshape(self.config.batch * self.config.context, -1)

    def memory_gb(self):
        used = C.c_double()
        self.check(self.lib.tg_memory(self.handle, C.byref(used)))
        return used.value

    def profile(self, reset=True):
        names = (C.c_char_p * 32)()
        ms = (C.c_double * 32)()
        launches = (C.c_int64 * 32)()
        n = self.check(self.lib.tg_ex_profile(self.handle, names, ms, launches, 32, int(reset)))
        return {names[i].decode(): (ms[i], launches[i]) for i in range(n)}


def save_checkpoint(path, config: ConfigEx, weights, momentum, variance, step, schedule: OneCycle,
                    train_seconds=0.0, final_loss_sums=None, final_loss_batches=0) -> None:
    """Writes the training state as a torch.load-able archive (the reference's checkpoint format plus
    the model dimensions)."""
    lib = load_library()
    arrays = [np.ascontiguousarray(a, dtype=np.float32) for a in (weights, momentum, variance)]
    sums = np.ascontiguousarray(final_loss_sums if final_loss_sums is not None else np.zeros(config.base.context),
                                dtype=np.float64)
    state = Checkpoint(arrays[0].ctypes.data, arrays[1].ctypes.data, arrays[2].ctypes.data, sums.ctypes.data, step,
                       final_loss_batches, train_seconds, schedule)
    if lib.tg_ex_save_checkpoint(str(path).encode(), C.byref(config), C.byref(state)) < 0:
        raise RuntimeError(lib.tg_error().decode())


def load_checkpoint(path, config: ConfigEx) -> dict:
    lib = load_library()
    count = lib.tg_ex_parameter_count(C.byref(config))
    if count < 0:
        raise RuntimeError(lib.tg_error().decode())
    arrays = [np.empty(count, np.float32) for _ in range(3)]
    sums = np.empty(config.base.context, np.float64)
    state = Checkpoint(arrays[0].ctypes.data, arrays[1].ctypes.data, arrays[2].ctypes.data, sums.ctypes.data)
    if lib.tg_ex_load_checkpoint(str(path).encode(), C.byref(config), C.byref(state)) < 0:
        raise RuntimeError(lib.tg_error().decode())
    schedule = OneCycle(state.scheduler.total_steps)
    for name, _ in OneCycle._fields_:
        setattr(schedule, name, getattr(state.scheduler, name))
    return dict(weights=arrays[0], momentum=arrays[1], variance=arrays[2], step=int(state.step), schedule=schedule,
                train_seconds=float(state.train_seconds), final_loss_sums=sums,
                final_loss_batches=int(state.final_loss_batches))


def require_matching_ranks(config: ConfigEx, all_gather) -> None:
    """Refuses to go on unless every rank of the job holds the same configuration (apart from rank and
    device).  ``all_gather(value: int) -> list[int]`` is the caller's own exchange (torch.distributed,
    MPI, a file): it must return every rank's value, in rank order, on every rank.  Call it before
    creating the engine: a communicator built from mismatched configurations hangs or trains garbage."""
    lib = load_library()
    digest = lib.tg_ex_config_digest(C.byref(config))
    if not digest:
        raise RuntimeError(lib.tg_error().decode())
    digests = list(all_gather(int(digest)))
    ranks = list(all_gather(int(config.rank)))
    if len(digests) != config.world or sorted(ranks) != list(range(config.world)):
        raise RuntimeError(f"data-parallel job: {len(digests)} ranks answered with ranks {ranks}, "
                           f"this configuration says world {config.world}")
    if len(set(digests)) != 1:
        different = [r for r, d in enumerate(digests) if d != digests[0]]
        raise RuntimeError(f"data-parallel job: ranks {different} hold a different configuration than rank 0")


def initialize_weights(config: ConfigEx) -> np.ndarray:
    """model.cpp:7-31 for any architecture."""
    lib = load_library()
    n = lib.tg_ex_parameter_count(C.byref(config))
    if n < 0:
        raise RuntimeError(lib.tg_error().decode())
    w = np.empty(n, np.float32)
    if lib.tg_ex_initialize_weights(C.byref(config), w.ctypes.data) < 0:
        raise RuntimeError(lib.tg_error().decode())
    return w


def parameter_layout(config: ConfigEx):
    lib = load_library()
    offsets, rows, cols = np.zeros(1024, np.int64), np.zeros(1024, np.int32), np.zeros(1024, np.int32)
    n = lib.tg_ex_parameter_layout(C.byref(config), offsets.ctypes.data, rows.ctypes.data, cols.ctypes.data, 1024)
    if n < 0:
        raise RuntimeError(lib.tg_error().decode())
    return [(int(offsets[i]), int(rows[i]), int(cols[i])) for i in range(n)]
