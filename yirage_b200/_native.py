"""ctypes binding of the C ABI in include/ypk.h.

The structures below mirror the header field by field.  Loading fails loudly when
libypk.so is missing: there is no Python or CPU fallback for the device path.
"""
import atexit
import ctypes as C
import os
import sys
import weakref

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libypk.so")

YPK_ABI_VERSION = 1

# enum ypk_error
YPK_OK, ERR_INVALID, ERR_CUDA, ERR_TIMEOUT, ERR_STATE, ERR_UNSUPPORTED = 0, -1, -2, -3, -4, -5

# enum ypk_dtype
F16, BF16, F32, I32, I64 = 940, 941, 942, 955, 965

# enum ypk_task_type
(TASK_NOP, TASK_EMBED, TASK_LINEAR, TASK_ATTENTION, TASK_ARGMAX_PARTIAL, TASK_ARGMAX_REDUCE,
 TASK_RMSNORM, TASK_SILU_MUL, TASK_ALLREDUCE, TASK_NGRAM_PARTIAL, TASK_NGRAM_GLOBAL,
 TASK_VERIFY, TASK_MOE_TOPK, TASK_MOE_SILU_MUL, TASK_MOE_COMBINE) = range(15)

TASK_NAMES = {
    TASK_NOP: "nop", TASK_EMBED: "embedding", TASK_LINEAR: "linear", TASK_ATTENTION: "attention",
    TASK_ARGMAX_PARTIAL: "argmax_partial", TASK_ARGMAX_REDUCE: "argmax_reduce",
    TASK_RMSNORM: "rmsnorm", TASK_SILU_MUL: "silu_mul", TASK_ALLREDUCE: "allreduce",
    TASK_NGRAM_PARTIAL: "find_ngram_partial", TASK_NGRAM_GLOBAL: "find_ngram_global",
    TASK_VERIFY: "target_verify_greedy", TASK_MOE_TOPK: "moe_topk_softmax",
    TASK_MOE_SILU_MUL: "moe_silu_mul", TASK_MOE_COMBINE: "moe_mul_sum_add",
}

F_NORM, F_RESIDUAL, F_SILU_MUL, F_F16, F_ROPE, F_NORM_NOWEIGHT = 0x1, 0x2, 0x4, 0x8, 0x10, 0x40
F_QK_NORM = 0x20
F_QTILES = 0x80
F_MOE = 0x4000
F_LL_IN, F_LL_RES, F_LL_OUT, F_LL_PUSH, F_LL_OPT = 0x100, 0x200, 0x400, 0x800, 0x1000
F_TRIG_WIDE = 0x2000
F_NORM_OUT, F_NORM_PRE = 0x8000, 0x10000

NPTR, NINT, NFLT = 8, 16, 4


def ref(slot, byte_off=0):
    """Encode a task operand: tensor slot + byte offset (YPK_REF in the header)."""
    assert 0 <= slot < 65534 and 0 <= byte_off < (1 << 48)
    return ((slot + 1) << 48) | byte_off


class Task(C.Structure):
    _fields_ = [
        ("type", C.c_int32), ("flags", C.c_uint32),
        ("dep_event", C.c_int32), ("dep_count", C.c_int32),
        ("trig_event", C.c_int32), ("op_id", C.c_int32),
        ("ptr", C.c_uint64 * NPTR),
        ("iarg", C.c_int32 * NINT),
        ("farg", C.c_float * NFLT),
        ("ptr_aux", C.c_uint64),
    ]


assert C.sizeof(Task) == 176


class Config(C.Structure):
    _fields_ = [
        ("abi_version", C.c_int32), ("device", C.c_int32),
        ("world_size", C.c_int32), ("rank", C.c_int32),
        ("num_workers", C.c_int32), ("mode", C.c_int32),
        ("max_seq_length", C.c_int32), ("max_num_batched_requests", C.c_int32),
        ("max_num_batched_tokens", C.c_int32), ("max_num_pages", C.c_int32),
        ("page_size", C.c_int32), ("total_num_requests", C.c_int32),
        ("eos_token_id", C.c_int64), ("wait_budget_ns", C.c_uint64),
        ("step", C.c_void_p), ("tokens", C.c_void_p), ("input_tokens", C.c_void_p),
        ("output_tokens", C.c_void_p), ("num_new_tokens", C.c_void_p),
        ("prompt_lengths", C.c_void_p), ("qo_indptr", C.c_void_p),
        ("paged_kv_indptr", C.c_void_p), ("paged_kv_indices", C.c_void_p),
        ("paged_kv_last_page_len", C.c_void_p),
        ("profiler_buffer", C.c_void_p), ("profiler_bytes", C.c_uint64),
    ]


class Status(C.Structure):
    _fields_ = [
        ("error", C.c_int32), ("fail_worker", C.c_int32), ("fail_task", C.c_int32),
        ("fail_event", C.c_int32), ("iterations", C.c_int64), ("finished", C.c_int32),
        ("active_tokens", C.c_int32), ("tasks_executed", C.c_int64),
        ("tensor_core_tasks", C.c_int64),
    ]


# Every symbol include/ypk.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "ypk_abi_version": (C.c_int, []),
    "ypk_last_error": (C.c_char_p, [C.c_void_p]),
    "ypk_create": (C.c_int, [C.POINTER(Config), C.POINTER(C.c_void_p)]),
    "ypk_destroy": (C.c_int, [C.c_void_p]),
    "ypk_bind_tensor": (C.c_int, [C.c_void_p, C.c_int32, C.c_char_p, C.c_void_p, C.c_uint64]),
    "ypk_alloc_tensor": (C.c_int, [C.c_void_p, C.c_int32, C.c_char_p, C.c_uint64]),
    "ypk_shuffle_tensor": (C.c_int, [C.c_void_p, C.c_int32, C.c_char_p, C.c_int32,
                                     C.POINTER(C.c_int32), C.POINTER(C.c_int32),
                                     C.POINTER(C.c_int32), C.c_uint64]),
    "ypk_comm_init": (C.c_int, [C.c_void_p, C.c_uint64]),
    "ypk_alloc_symmetric": (C.c_int, [C.c_void_p, C.c_int32, C.c_char_p, C.c_uint64]),
    "ypk_comm_export": (C.c_int, [C.c_void_p, C.c_void_p]),
    "ypk_comm_import": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p]),
    "ypk_tensor_ptr": (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(C.c_void_p),
                                 C.POINTER(C.c_uint64)]),
    "ypk_read_tensor": (C.c_int, [C.c_void_p, C.c_int32, C.c_uint64, C.c_void_p, C.c_uint64]),
    "ypk_load_graph": (C.c_int, [C.c_void_p, C.POINTER(Task), C.c_int32, C.c_int32,
                                 C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.c_int32]),
    "ypk_reset": (C.c_int, [C.c_void_p]),
    "ypk_launch": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32]),
    "ypk_launch_async": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32]),
    "ypk_wait": (C.c_int, [C.c_void_p]),
    "ypk_get_status": (C.c_int, [C.c_void_p, C.POINTER(Status)]),
    "ypk_set_pause_below": (C.c_int, [C.c_void_p, C.c_int32]),
    "ypk_adopt_batch": (C.c_int, [C.c_void_p, C.c_void_p]),
    "ypk_argmax_noalloc": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int64, C.c_void_p,
                                     C.c_void_p]),
    "ypk_transpose_16bit": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
}

_lib = None


class YpkError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"ypk error {code}: {message}")
        self.code = code


def load():
    """dlopen libypk.so and declare the prototypes.  Raises if the library is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m yirage_b200.build` "
            "(there is no fallback implementation)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if lib.ypk_abi_version() != YPK_ABI_VERSION:
        raise ImportError("libypk.so ABI version mismatch; rebuild it")
    _lib = lib
    return lib


def check(handle, rc):
    if rc != YPK_OK:
        msg = load().ypk_last_error(handle)
        raise YpkError(rc, msg.decode() if msg else "")


_live = weakref.WeakSet()


@atexit.register
def _close_all():
    # handles are destroyed here, while the library is still loaded, rather than from
    # __del__ during interpreter teardown
    for h in list(_live):
        h.close()


class Handle:
    """Thin RAII wrapper over ypk_handle."""

    def __init__(self, cfg: Config):
        self.lib = load()
        self._h = C.c_void_p()
        cfg.abi_version = YPK_ABI_VERSION
        check(None, self.lib.ypk_create(C.byref(cfg), C.byref(self._h)))
        self.cfg = cfg
        _live.add(self)

    @property
    def raw(self):
        return self._h

    def bind(self, slot, name, ptr, nbytes):
        check(self._h, self.lib.ypk_bind_tensor(self._h, slot, name.encode(), C.c_void_p(ptr), nbytes))

    def alloc(self, slot, name, nbytes):
        check(self._h, self.lib.ypk_alloc_tensor(self._h, slot, name.encode(), nbytes))

    def comm_init(self, nbytes):
        check(self._h, self.lib.ypk_comm_init(self._h, nbytes))

    def alloc_symmetric(self, slot, name, nbytes):
        check(self._h, self.lib.ypk_alloc_symmetric(self._h, slot, name.encode(), nbytes))

    def comm_export(self) -> bytes:
        buf = C.create_string_buffer(64)
        check(self._h, self.lib.ypk_comm_export(self._h, buf))
        return buf.raw

    def comm_import(self, peer, handle: bytes):
        check(self._h, self.lib.ypk_comm_import(self._h, peer, C.c_char_p(handle)))

    def shuffle(self, dst_slot, name, src_slots, rows, gran, row_bytes):
        n = len(src_slots)
        arr = C.c_int32 * n
        check(self._h, self.lib.ypk_shuffle_tensor(self._h, dst_slot, name.encode(), n,
                                                   arr(*src_slots), arr(*rows), arr(*gran),
                                                   row_bytes))

    def tensor_ptr(self, slot):
        p, b = C.c_void_p(), C.c_uint64()
        check(self._h, self.lib.ypk_tensor_ptr(self._h, slot, C.byref(p), C.byref(b)))
        return p.value, b.value

    def read_tensor(self, slot, byte_off, dst_ptr, nbytes):
        check(self._h, self.lib.ypk_read_tensor(self._h, slot, byte_off, C.c_void_p(dst_ptr), nbytes))

    def load_graph(self, tasks, num_events, queue, queue_off):
        n = len(tasks)
        tarr = (Task * n)(*tasks)
        qarr = (C.c_int32 * len(queue))(*queue)
        oarr = (C.c_int32 * len(queue_off))(*queue_off)
        check(self._h, self.lib.ypk_load_graph(self._h, tarr, n, num_events, qarr, oarr,
                                               len(queue_off) - 1))

    def reset(self):
        check(self._h, self.lib.ypk_reset(self._h))

    def launch(self, stream=0, max_iterations=0, batch=1):
        check(self._h, self.lib.ypk_launch(self._h, C.c_void_p(stream), max_iterations, batch))

    def launch_async(self, stream=0, max_iterations=0, batch=1):
        check(self._h, self.lib.ypk_launch_async(self._h, C.c_void_p(stream), max_iterations, batch))

    def wait(self):
        check(self._h, self.lib.ypk_wait(self._h))

    def set_pause_below(self, tokens: int):
        check(self._h, self.lib.ypk_set_pause_below(self._h, tokens))

    def adopt_batch(self, src: "Handle"):
        check(self._h, self.lib.ypk_adopt_batch(self._h, src._h))

    def status(self):
        st = Status()
        check(self._h, self.lib.ypk_get_status(self._h, C.byref(st)))
        return st

    def close(self):
        if self._h:
            self.lib.ypk_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        if sys.is_finalizing():
            return
        try:
            self.close()
        except Exception:
            pass
