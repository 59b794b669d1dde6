"""ctypes binding of libxlstm_b200.so. Raises at import when the library is absent."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libxlstm_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        "libxlstm_b200.so is not built (expected at %s). Run `python neural-networks_b200/build.py`; "
        "this engine has no CPU or eager fallback." % LIB_PATH)

lib = ctypes.CDLL(LIB_PATH)

OK, DECLINED = 0, 1
F32, BF16 = 0, 1
FORCE_SIMT = 1
PACK_SHORT = 2


class MlstmShape(ctypes.Structure):
    _fields_ = [("B", ctypes.c_int), ("H", ctypes.c_int), ("T", ctypes.c_int), ("dqk", ctypes.c_int),
                ("dhv", ctypes.c_int), ("L", ctypes.c_int), ("dtype", ctypes.c_int), ("gdtype", ctypes.c_int),
                ("flags", ctypes.c_uint)]


class SlstmSlabs(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in
                ("c_prev", "n_prev", "ipr", "fpr", "c", "n", "zt", "ot", "h_prev")]


class AdamwDesc(ctypes.Structure):
    _fields_ = [("p", ctypes.c_void_p), ("g", ctypes.c_void_p), ("m", ctypes.c_void_p), ("v", ctypes.c_void_p),
                ("p_bf16", ctypes.c_void_p), ("len", ctypes.c_uint64), ("wd", ctypes.c_float), ("_pad", ctypes.c_float)]


_vp, _i, _u, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_float, ctypes.c_size_t
_shape_p = ctypes.POINTER(MlstmShape)

SIGNATURES = {
    "xlstm_version": (ctypes.c_int, []),
    "xlstm_last_error": (ctypes.c_char_p, []),
    "xlstm_launch_count": (ctypes.c_uint64, []),
    "xlstm_device_status": (ctypes.c_int, []),
    "xlstm_mlstm_saved_bytes": (_sz, [_shape_p]),
    "xlstm_mlstm_fw_workspace_bytes": (_sz, [_shape_p]),
    "xlstm_mlstm_bw_workspace_bytes": (_sz, [_shape_p, _i]),
    "xlstm_mlstm_fw": (_i, [_vp, _shape_p] + [_vp] * 17 + [_sz]),
    "xlstm_mlstm_final_state": (_i, [_vp, _shape_p] + [_vp] * 11),
    "xlstm_mlstm_bw": (_i, [_vp, _shape_p] + [_vp] * 24 + [_sz]),
    "xlstm_slstm_fw": (_i, [_vp] * 9 + [ctypes.POINTER(SlstmSlabs), _i, _i, _i, _i, _i, _u]),
    "xlstm_slstm_bw": (_i, [_vp] * 7 + [ctypes.POINTER(SlstmSlabs), _i, _i, _i, _i, _i, _u]),
    "xlstm_rmsnorm_fw": (_i, [_vp, _vp, _i, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _f]),
    "xlstm_rmsnorm_bw_workspace_bytes": (_sz, [_i, _i]),
    "xlstm_rmsnorm_bw": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _vp, _sz]),
    "xlstm_ce_workspace_bytes": (_sz, [_i]),
    "xlstm_ce_fw_bw": (_i, [_vp] * 6 + [_i, _i, _f, _vp, _sz]),
    "xlstm_ce_fw_bw_noalloc": (_i, [_vp] * 6 + [_i, _i, _f]),
    "xlstm_softcap_ce_fw_bw": (_i, [_vp] * 6 + [_i, _i, _f, _f, _vp, _sz]),
    "xlstm_swiglu_fw": (_i, [_vp] * 3 + [_i, _vp, _vp, _i, _vp, _i, _sz]),
    "xlstm_swiglu_bw": (_i, [_vp, _vp, _i, _vp, _vp, _i, _vp, _vp, _i, _vp, _vp, _i, _sz]),
    "xlstm_ogate_fw": (_i, [_vp] * 4 + [_i, _vp, _i, _sz]),
    "xlstm_ogate_bw": (_i, [_vp] * 5 + [_i, _vp, _sz]),
    "xlstm_colsum_workspace_bytes": (_sz, [_i, _i]),
    "xlstm_colsum_narrow": (_i, [_vp, _vp, _i, _i, _i, _f, _vp, _vp, _vp, _sz]),
    "xlstm_bias_rows": (_i, [_vp, _vp, _vp, _vp, _i, _i]),
    "xlstm_embedding_scatter_add": (_i, [_vp] * 5 + [_i, _i]),
    "xlstm_split3_bf16": (_i, [_vp] * 5 + [_sz]),
    "xlstm_adamw_multi": (_i, [_vp, ctypes.POINTER(AdamwDesc), _i, _f, _f, _f, _f, _f, _f, _i]),
    "xlstm_dp_unique_id": (_i, [_vp]),
    "xlstm_dp_init": (_i, [_i, _i, _vp]),
    "xlstm_dp_init_comm": (_i, [_vp]),
    "xlstm_dp_world": (_i, []),
    "xlstm_dp_bucket_register": (_i, [_vp, _sz]),
    "xlstm_dp_bucket_start": (_i, [_i, _vp]),
    "xlstm_dp_wait": (_i, [_vp]),
    "xlstm_dp_shutdown": (_i, []),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)  # AttributeError here means the library does not match the header
    _fn.restype = _res
    _fn.argtypes = _args


class XlstmError(RuntimeError):
    pass


class Declined(XlstmError):
    """The engine does not cover this shape; nothing was launched."""


def check(rc, what):
    if rc == OK:
        return
    msg = lib.xlstm_last_error().decode("utf-8", "replace")
    if rc == DECLINED:
        raise Declined("%s declined: %s" % (what, msg))
    raise XlstmError("%s failed (%d): %s" % (what, rc, msg))
