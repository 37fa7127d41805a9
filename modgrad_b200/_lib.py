"""ctypes binding of libmodgrad_cuda.so.  There is no fallback: a missing library raises."""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "lib" / "libmodgrad_cuda.so"
HEADER = PKG.parent / "include" / "modgrad_cuda.h"

_lib = None

vp, sz, ci, cf = C.c_void_p, C.c_size_t, C.c_int, C.c_float

# name -> (restype, argtypes).  Every function include/modgrad_cuda.h declares is listed.
SIGNATURES = {
    "mg_get_device_count": (ci, [C.POINTER(ci)]),
    "mg_set_device": (ci, [ci]),
    "mg_malloc": (ci, [C.POINTER(vp), sz]),
    "mg_free": (ci, [vp]),
    "mg_memcpy_h2d": (ci, [vp, vp, sz]),
    "mg_memcpy_d2h": (ci, [vp, vp, sz]),
    "mg_memcpy_d2d": (ci, [vp, vp, sz]),
    "mg_memset": (ci, [vp, ci, sz]),
    "mg_device_synchronize": (ci, []),
    "mg_mem_get_info": (ci, [C.POINTER(sz), C.POINTER(sz)]),
    "mg_get_error_string": (C.c_char_p, [ci]),
    "mg_version": (C.c_char_p, []),
    "launch_matvec_q4k": (ci, [vp, vp, vp, ci, ci]),
    "launch_matvec_q4k_on_stream": (ci, [vp, vp, vp, ci, ci, vp]),
    "launch_matvec_q4k_noalloc_on_stream": (ci, [vp, vp, vp, ci, ci, vp]),
    "launch_quantize_q8_1": (ci, [vp, vp, vp, vp, ci]),
    "launch_quantize_q8_1_on_stream": (ci, [vp, vp, vp, vp, ci, vp]),
    "launch_matvec_q4k_dp4a": (ci, [vp, vp, vp, vp, vp, ci, ci]),
    "launch_matvec_q4k_dp4a_on_stream": (ci, [vp, vp, vp, vp, vp, ci, ci, vp]),
    "launch_matvec_q5k": (ci, [vp, vp, vp, ci, ci]),
    "launch_matvec_q5k_on_stream": (ci, [vp, vp, vp, ci, ci, vp]),
    "launch_matvec_q6k": (ci, [vp, vp, vp, ci, ci]),
    "launch_matvec_q6k_on_stream": (ci, [vp, vp, vp, ci, ci, vp]),
    "launch_matvec_q6k_dp4a": (ci, [vp, vp, vp, vp, vp, ci, ci]),
    "launch_matvec_q6k_dp4a_on_stream": (ci, [vp, vp, vp, vp, vp, ci, ci, vp]),
    "mg_dequant_q5k_on_stream": (ci, [vp, ci, vp, vp]),
    "mg_dequant_q6k_on_stream": (ci, [vp, ci, vp, vp]),
    "launch_dequant_q4k": (ci, [vp, ci, vp]),
    "launch_dequant_q4k_on_stream": (ci, [vp, ci, vp, vp]),
    "mg_matvec_q4k_bias_on_stream": (ci, [vp, vp, vp, vp, ci, ci, vp]),
    "mg_q4k_limb_record_bytes": (sz, [ci]),
    "mg_matvec_q4k_timeouts": (C.c_longlong, []),
    "mg_matvec_q4k_speculation": (ci, [ci]),
    "mg_pdl_early_trigger": (ci, [ci]),
    "mg_peer_exchange_create": (ci, [sz, ci, ci, vp, C.POINTER(vp)]),
    "mg_peer_exchange_open": (ci, [vp, vp]),
    "mg_peer_arena": (vp, [vp]),
    "mg_peer_arena_offset": (sz, []),
    "mg_peer_fuse_next": (ci, [vp, ci]),
    "mg_peer_gather_on_stream": (ci, [vp, ci, sz, sz, sz, vp]),
    "mg_peer_exchange_status": (ci, [vp]),
    "mg_peer_exchange_set_spin_limit": (ci, [vp, C.c_uint]),
    "mg_decoder_set_exchange_spin_limit": (ci, [vp, C.c_uint]),
    "mg_peer_exchange_destroy": (None, [vp]),
    "mg_q4k_x_to_limbs_on_stream": (ci, [vp, ci, vp, vp]),
    "mg_matvec_q4k_limbs_on_stream": (ci, [vp, vp, vp, vp, ci, ci, vp]),
    "mg_matvec_q4k_multi_on_stream": (ci, [ci, vp, vp, ci, vp, vp, vp, ci, vp]),
    "mg_rmsnorm_matvec_q4k_multi_on_stream": (ci, [ci, vp, vp, vp, cf, vp, vp, vp, ci, vp]),
    "mg_swiglu_limbs_on_stream": (ci, [vp, vp, vp, ci, vp, vp]),
    "mg_matmul_q4k_scratch_bytes": (sz, [ci, ci]),
    "launch_matmul_q4k_on_stream": (ci, [vp, vp, vp, ci, ci, ci, vp, vp]),
    "mg_matmul_q4k_status": (ci, [vp, ci, ci]),
    "launch_rms_norm": (ci, [vp, vp, vp, ci, ci, cf]),
    "launch_rms_norm_on_stream": (ci, [vp, vp, vp, ci, ci, cf, vp]),
    "launch_residual_add": (ci, [vp, vp, ci]),
    "launch_residual_add_on_stream": (ci, [vp, vp, ci, vp]),
    "launch_scale": (ci, [vp, cf, ci]),
    "launch_scale_on_stream": (ci, [vp, cf, ci, vp]),
    "launch_geglu": (ci, [vp, vp, vp, ci]),
    "launch_geglu_on_stream": (ci, [vp, vp, vp, ci, vp]),
    "launch_swiglu": (ci, [vp, vp, vp, ci]),
    "launch_swiglu_on_stream": (ci, [vp, vp, vp, ci, vp]),
    "launch_softcap": (ci, [vp, cf, ci]),
    "launch_softcap_on_stream": (ci, [vp, cf, ci, vp]),
    "launch_rope_neox": (ci, [vp, ci, ci, ci, cf, vp]),
    "launch_rope_neox_on_stream": (ci, [vp, ci, ci, ci, cf, vp, vp]),
    "launch_copy": (ci, [vp, vp, ci]),
    "launch_copy_on_stream": (ci, [vp, vp, ci, vp]),
    "launch_sdpa_decode": (ci, [vp, vp, vp, vp, ci, ci, ci, ci, ci, cf, ci]),
    "launch_sdpa_decode_flash": (ci, [vp, vp, vp, vp, ci, ci, ci, ci, ci, cf, ci]),
    "launch_sdpa_decode_on_stream": (ci, [vp, vp, vp, vp, ci, ci, ci, ci, ci, cf, ci, vp]),
    "launch_sdpa_decode_flash_on_stream": (ci, [vp, vp, vp, vp, ci, ci, ci, ci, ci, cf, ci, vp]),
    "mg_sdpa_f16kv_scratch_bytes": (sz, [ci, ci, ci]),
    "mg_sdpa_decode_f16kv_on_stream": (ci, [vp, vp, vp, vp, ci, ci, ci, ci, vp, cf, vp, ci, vp]),
    "mg_rope_kv_append_f16_on_stream": (ci, [vp, vp, vp, vp, vp, ci, vp, ci, ci, ci, cf, vp, vp]),
    "mg_sdpa_rope_f16kv_scratch_bytes": (sz, [ci, ci, ci, ci]),
    "mg_sdpa_rope_decode_f16kv_on_stream": (ci, [vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, vp, cf, cf, vp, vp, ci, vp]),
    "mg_matvec_f16_on_stream": (ci, [vp, vp, vp, ci, ci, vp]),
    "mg_embed_f16_on_stream": (ci, [vp, ci, vp, vp, ci, ci, vp]),
    "mg_argmax_on_stream": (ci, [vp, ci, vp, vp, vp, vp, vp]),
    "mg_decoder_create": (ci, [vp, C.POINTER(vp)]),
    "mg_decoder_create_typed": (ci, [vp, vp, ci, ci, C.POINTER(vp)]),
    "mg_decoder_create_typed_sharded": (ci, [vp, vp, ci, ci, ci, ci, vp, C.POINTER(vp)]),
    "mg_decoder_weight_type": (ci, [vp, ci, ci]),
    "mg_matvec_kquant_on_stream": (ci, [ci, vp, vp, ci, vp, vp, ci, ci, vp]),
    "mg_rmsnorm_matvec_kquant_on_stream": (ci, [ci, vp, vp, vp, C.c_float, vp, ci, ci, vp]),
    "mg_embed_kquant_on_stream": (ci, [vp, ci, ci, vp, vp, ci, ci, vp]),
    "mg_nccl_unique_id": (ci, [vp]),
    "mg_decoder_shard_ranges": (ci, [vp, ci, ci, vp]),
    "mg_decoder_create_sharded": (ci, [vp, ci, ci, vp, C.POINTER(vp)]),
    "mg_decoder_destroy": (None, [vp]),
    "mg_decoder_last_error": (C.c_char_p, [vp]),
    "mg_decoder_upload": (ci, [vp, ci, ci, vp, sz]),
    "mg_decoder_set_kv": (ci, [vp, ci, vp, vp, ci]),
    "mg_decoder_set_position": (ci, [vp, ci]),
    "mg_decoder_forward_token": (ci, [vp, ci, vp, vp]),
    "mg_decoder_generate": (ci, [vp, ci, ci, vp, vp]),
    "mg_decoder_buffer": (vp, [vp, ci]),
    "mg_decoder_kernels_per_token": (ci, [vp]),
    "mg_decoder_gather_mode": (ci, [vp]),
    "mg_decoder_weight_arena": (vp, [vp, C.POINTER(sz)]),
    "mg_decoder_weight_ptr": (vp, [vp, ci, ci]),
    "mg_quantize_row_q4_k": (ci, [vp, vp, sz]),
    "mg_linear_q4k_from_f32": (ci, [vp, vp, ci, ci, C.POINTER(vp)]),
    "mg_linear_q4k_from_blocks": (ci, [vp, vp, ci, ci, C.POINTER(vp)]),
    "mg_linear_q4k_destroy": (None, [vp]),
    "mg_linear_q4k_set_expanded": (ci, [vp, ci]),
    "mg_linear_q4k_is_resident": (ci, [vp]),
    "mg_linear_q4k_host_size_bytes": (sz, [vp]),
    "mg_linear_q4k_device_size_bytes": (sz, [vp]),
    "mg_linear_q4k_host_blocks": (vp, [vp, C.POINTER(sz)]),
    "mg_linear_q4k_ensure_resident": (ci, [vp, vp]),
    "mg_linear_q4k_evict": (None, [vp]),
    "mg_linear_q4k_forward": (ci, [vp, vp, vp, ci, vp]),
    "mg_matvec_f32_on_stream": (ci, [vp, vp, vp, vp, ci, ci, vp]),
    "mg_gguf_open": (ci, [C.c_char_p, C.POINTER(vp)]),
    "mg_gguf_parse_memory": (ci, [vp, sz, C.POINTER(vp)]),
    "mg_gguf_close": (None, [vp]),
    "mg_gguf_last_error": (C.c_char_p, []),
    "mg_gguf_version": (ci, [vp]),
    "mg_gguf_data_offset": (sz, [vp]),
    "mg_gguf_n_tensors": (ci, [vp]),
    "mg_gguf_n_meta": (ci, [vp]),
    "mg_gguf_find_tensor": (ci, [vp, C.c_char_p]),
    "mg_gguf_tensor": (ci, [vp, ci, C.POINTER(C.c_char_p), C.POINTER(ci), C.POINTER(C.c_uint64), C.POINTER(C.c_uint32),
                             C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "mg_gguf_tensor_data": (vp, [vp, ci]),
    "mg_gguf_meta_u32": (ci, [vp, C.c_char_p, C.POINTER(C.c_uint32)]),
    "mg_gguf_meta_f32": (ci, [vp, C.c_char_p, C.POINTER(cf)]),
    "mg_gguf_meta_str": (C.c_char_p, [vp, C.c_char_p]),
    "mg_gguf_meta_array_len": (C.c_longlong, [vp, C.c_char_p]),
    "mg_gguf_block_size": (None, [C.c_uint32, C.POINTER(sz), C.POINTER(sz)]),
    "mg_decoder_config_from_gguf": (ci, [vp, ci, vp]),
    "mg_decoder_load_gguf": (ci, [C.c_char_p, ci, ci, ci, vp, C.POINTER(vp)]),
    "mg_decoder_load_error": (C.c_char_p, []),
    "mg_backend_create": (ci, [ci, C.POINTER(vp)]),
    "mg_backend_destroy": (None, [vp]),
    "mg_backend_name": (C.c_char_p, [vp]),
    "mg_backend_device_info": (C.c_char_p, [vp]),
    "mg_backend_last_error": (C.c_char_p, [vp]),
    "mg_backend_supports_matvec": (ci, [vp, vp, sz, vp, sz, vp, sz, vp, sz, sz, sz, ci]),
    "mg_backend_dispatch_matvec": (ci, [vp, vp, sz, vp, sz, vp, sz, vp, sz, sz, sz, ci]),
    "mg_backend_supports_dequant_q4k_resident": (ci, [vp, vp, vp, sz]),
    "mg_backend_dispatch_dequant_q4k_resident": (ci, [vp, vp, vp, sz]),
    "mg_backend_invalidate_cache": (None, [vp]),
    "mg_backend_cached_weights": (sz, [vp]),
    "mg_buffer_matvec_q4k": (ci, [vp, sz, vp, vp, sz, sz]),
    "mg_buffer_matvec_q4k_into": (ci, [vp, vp, vp, sz, sz]),
}


def declared_symbols(header: Path = HEADER) -> list[str]:
    """Function names declared in the C header (what the library must export)."""
    text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b((?:launch|mg)_[a-z0-9_]+)\s*\(", text)))


def load() -> C.CDLL:
    """Load the CUDA library; raise (never fall back) when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m modgrad_b200.build` "
            "(there is no CPU or PyTorch fallback for the Q4_K path)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header/library mismatch: fail loudly
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
