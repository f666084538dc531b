"""ctypes binding of libcrucible_attn.so, one Structure per struct of include/crucible_attn.h."""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libcrucible_attn.so")

OK, ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_TIMEOUT = range(5)
OUT_RAW_F32, OUT_RAW_BF16, OUT_EXL3_WHT = range(3)
IN_F32, IN_BF16 = range(2)
GDN_SERIAL_F32, GDN_CHUNK_TC = range(2)
PEND_FLOATS, QSA_PART, QSA_SPLITS, SEL_BLOCKS, MAX_STEP_ROWS = 258, 258, 32, 512, 13


class CrError(RuntimeError):
    def __init__(self, status, text):
        super().__init__("crucible_attn status %d: %s" % (status, text))
        self.status = status


class Geometry(C.Structure):
    _fields_ = [("hidden", C.c_int), ("q_heads", C.c_int), ("kv_heads", C.c_int),
                ("gdn_vheads", C.c_int), ("gdn_kheads", C.c_int)]

    @property
    def gdn_channels(self):
        return 2 * self.gdn_kheads * 128 + self.gdn_vheads * 128


GEOM_BENCH = Geometry(2048, 16, 2, 32, 16)
GEOM_REF = Geometry(2560, 24, 2, 48, 16)

P = C.c_void_p


class Options(C.Structure):
    _fields_ = [("gdn_part_chunks", C.c_int), ("pdl", C.c_int), ("qsa_score_simt", C.c_int), ("qsa_union_rows", C.c_int)]


class Span(C.Structure):
    _fields_ = [("ptr", P), ("bytes", C.c_size_t)]


class ProjOut(C.Structure):
    _fields_ = [("ptr", P), ("col0", C.c_int), ("cols", C.c_int), ("ld", C.c_int), ("f32", C.c_int)]


class GdnArgs(C.Structure):
    _fields_ = [("qkv", P), ("z", P), ("x", P), ("ab", P), ("conv", P), ("A_log", P), ("dt_bias", P),
                ("gamma", P), ("hist", P), ("state", P), ("suh_out", P), ("out", P), ("pend", P),
                ("pos0", C.c_int), ("R", C.c_int), ("replay", C.c_int), ("commit", C.c_int),
                ("pack_rows", C.c_int), ("pack_off", C.c_int)]


class GdnPrefillArgs(C.Structure):
    _fields_ = [("input", GdnArgs), ("ab_logits", P), ("in_dtype", C.c_int), ("workspace", P),
                ("workspace_bytes", C.c_size_t), ("raw_y", P)]


class QsaCache(C.Structure):
    _fields_ = [("k", P), ("v", P), ("ik_raw", P), ("ik_pool", P), ("raw_slots", C.c_int)]


class QsaArgs(C.Structure):
    _fields_ = [("q", P), ("k", P), ("v", P), ("idx", P), ("q_norm1", P), ("k_norm1", P), ("iq_norm1", P),
                ("ik_norm1", P), ("c", QsaCache), ("scores", P), ("sstride", C.c_int), ("sel", P), ("nsel", P),
                ("suh_o", P), ("out", P), ("pos0", C.c_int), ("R", C.c_int), ("context", P),
                ("pack_rows", C.c_int), ("pack_off", C.c_int), ("mrope", P), ("rope", P)]


class QsaUnion(C.Structure):
    _fields_ = [("list", P), ("count", P)]


class QsaPrefillArgs(C.Structure):
    _fields_ = [("input", QsaArgs), ("q_hi", P), ("scratch", P), ("scratch_bytes", C.c_size_t)]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError("libcrucible_attn.so is not built: run `python -m crucible_strix_halo_b200.build` "
                          "(there is no CPU fallback)")
    return C.CDLL(LIB_PATH)


lib = _load()
G = C.POINTER(Geometry)
_protos = {
    "cr_gdn_step": (C.c_int, [G, C.POINTER(GdnArgs), C.c_int, C.c_int, C.c_int, P]),
    "cr_gdn_prefill_workspace_bytes": (C.c_size_t, [G, C.c_int]),
    "cr_gdn_algo_available": (C.c_int, [C.c_int]),
    "cr_gdn_prefill_parts": (C.c_int, [C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int]),
    "cr_gdn_prefill": (C.c_int, [G, C.POINTER(GdnPrefillArgs), C.c_int, C.c_int, P]),
    "cr_gdn_materialize": (C.c_int, [G, C.POINTER(P), C.c_int, P]),
    "cr_qsa_scratch_bytes": (C.c_size_t, [G, C.c_int]),
    "cr_qsa_select_scratch_bytes": (C.c_size_t, [G, C.c_int]),
    "cr_qsa_pool_floats": (C.c_size_t, [C.c_int]),
    "cr_qsa_cache_bytes": (C.c_int, [G, C.c_int, C.c_int, C.POINTER(C.c_size_t)]),
    "cr_rope_table_fill": (C.c_int, [P, P]),
    "cr_rope_table_fill_yarn": (C.c_int, [P, C.c_int, P]),
    "cr_qsa_prep_queries": (C.c_int, [G, C.POINTER(QsaArgs), C.c_int, P]),
    "cr_qsa_prep": (C.c_int, [G, C.POINTER(QsaArgs), C.c_int, P]),
    "cr_qsa_select": (C.c_int, [G, C.POINTER(QsaArgs), C.c_int, P, C.c_size_t, P]),
    "cr_qsa_attn": (C.c_int, [G, C.POINTER(QsaArgs), C.c_int, P, C.c_size_t, C.c_int, P]),
    "cr_qsa_attn_static": (C.c_int, [G, C.POINTER(QsaArgs), C.c_int, C.c_int, P]),
    "cr_qsa_step": (C.c_int, [G, C.POINTER(QsaArgs), C.c_int, P, C.c_size_t, C.c_int, P]),
    "cr_qsa_prefill_scratch_bytes": (C.c_size_t, [G, C.c_int]),
    "cr_qsa_prefill_cache": (C.c_int, [G, C.POINTER(QsaArgs), P]),
    "cr_qsa_prefill": (C.c_int, [G, C.POINTER(QsaPrefillArgs), C.c_int, C.c_int, P]),
    "cr_qsa_prefill_attend": (C.c_int, [G, C.POINTER(QsaPrefillArgs), C.c_int, C.c_int, P]),
    "cr_qsa_union_list_ints": (C.c_size_t, [G, C.c_int]),
    "cr_qsa_union_tile_rows": (C.c_int, [G]),
    "cr_qsa_union_build": (C.c_int, [G, C.POINTER(QsaArgs), C.POINTER(QsaUnion), P]),
    "cr_qsa_shard_candidates": (C.c_int, [G, C.POINTER(QsaArgs), C.c_int, C.c_int, P, P, P]),
    "cr_qsa_shard_select": (C.c_int, [G, C.POINTER(QsaArgs), C.c_int, C.c_int, P, P, P]),
    "cr_qsa_merge_candidates": (C.c_int, [G, C.POINTER(QsaArgs), C.c_int, P, P, P]),
    "cr_qsa_shard_attn": (C.c_int, [G, C.POINTER(QsaArgs), C.c_int, C.c_int, P, P, C.c_size_t, P]),
    "cr_qsa_merge_partials": (C.c_int, [G, C.POINTER(QsaArgs), C.c_int, P, C.c_int, P]),
    "cr_proj_gemm": (C.c_int, [P, P, C.c_int, C.c_int, C.c_int, C.POINTER(ProjOut), C.c_int, P]),
    "cr_spans_bytes": (C.c_size_t, [C.POINTER(Span), C.c_int]),
    "cr_state_save": (C.c_int, [C.POINTER(Span), C.c_int, P, C.c_size_t, P]),
    "cr_state_restore": (C.c_int, [C.POINTER(Span), C.c_int, P, C.c_size_t, P]),
    "cr_debug_umma_gemm": (C.c_int, [P, P, P, C.c_int, C.c_int, P, P]),
    "cr_debug_umma_f16_gemm": (C.c_int, [P, P, P, C.c_int, C.c_int, C.c_int, P, P]),
    "cr_debug_umma_kv_step": (C.c_int, [P, P, C.c_int, C.c_int, C.c_int, P, P, P, P, P, P, P]),
    "cr_last_error": (C.c_char_p, []),
    "cr_version": (C.c_int, []),
    "cr_device_status": (C.c_int, []),
    "cr_device_check": (C.c_int, []),
    "cr_device_status_clear": (C.c_int, []),
    "cr_get_options": (C.c_int, [C.POINTER(Options)]),
    "cr_set_options": (C.c_int, [C.POINTER(Options)]),
    "cr_debug_wait_timeout": (C.c_int, [P, C.c_uint, P]),
    "cr_kernel_launches": (C.c_ulonglong, []),
    "cr_profile_enable": (C.c_int, [C.c_int]),
    "cr_profile_begin": (C.c_int, [P]),
    "cr_profile_collect": (C.c_int, [C.c_char_p, C.POINTER(C.c_float), C.POINTER(C.c_int), C.c_int]),
}
EXPORTS = tuple(_protos)
for _name, (_res, _args) in _protos.items():
    _fn = getattr(lib, _name)        # AttributeError here = the library lacks a declared symbol
    _fn.restype, _fn.argtypes = _res, _args


def get_options():
    o = Options()
    check(lib.cr_get_options(C.byref(o)))
    return o


def set_options(**kw):
    """Changes the named fields of the process-wide options and returns the previous values."""
    old = get_options()
    new = Options(old.gdn_part_chunks, old.pdl, old.qsa_score_simt, old.qsa_union_rows)
    for k, v in kw.items():
        setattr(new, k, v)
    check(lib.cr_set_options(C.byref(new)))
    return old


def check(status):
    if status != OK:
        raise CrError(status, lib.cr_last_error().decode())


def dptr(t):
    """Device (or host) address of a torch tensor, or None."""
    return None if t is None else C.c_void_p(t.data_ptr())


def profile_collect(max_stages=64):
    """{kernel name: (total ms, launches)} since the last collect (needs cr_profile_enable(1))."""
    names = C.create_string_buffer(32 * max_stages)
    ms = (C.c_float * max_stages)()
    calls = (C.c_int * max_stages)()
    n = lib.cr_profile_collect(names, ms, calls, max_stages)
    return {names.raw[32 * i:32 * i + 32].split(b"\0")[0].decode(): (ms[i], calls[i]) for i in range(n)}
