"""ctypes binding of libtgis_engine.so (C ABI: include/tgis_engine.h, include/tgis_kernels.h).

This is the reference-side binding a maintainer would add next to `build_async_engine_client`
(/root/reference/src/vllm_tgis_adapter/__main__.py:48); see INTEGRATION.md.  There is no Python/CPU fallback: if the
library is missing it is built with nvcc, and if that is impossible the import fails loudly.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

ABI_VERSION = 11
ARCH_LLAMA, ARCH_OPT, ARCH_PONENEX, ARCH_FALERAX, ARCH_REVEPEL, ARCH_SIKAZEN = 0, 1, 2, 3, 4, 5
MIXER_LATENT_ATTENTION, MIXER_PARALLEL, MIXER_SELECTIVE_SCAN, MIXER_WKV = 1, 2, 3, 4
MIXER_SIGMOID_ATTENTION, MIXER_SSD, MIXER_CHANNEL_DELTA = 5, 6, 7
MIXER_POOLED_ATTENTION, MIXER_HGRN = 8, 9
MLP_NONE, MLP_MOE, MLP_DENSE_GELU, MLP_MOE_SIGMOID, MLP_DENSE_SILU = 0, 1, 2, 3, 4
LAYER_ROT_INTERLEAVED, LAYER_SINK, LAYER_NO_OUT_GATE, LAYER_QKV_BIAS, LAYER_UNIT_QK = 1, 2, 4, 8, 16
STYLE_POST_NORM, STYLE_TIED_HEAD, STYLE_PARALLEL_GATED, STYLE_PARALLEL_PAIR = 1, 2, 4, 8
DTYPE_BF16, DTYPE_F32 = 0, 1
MAX_REQUEST_ID = 96
MAX_TOPN = 12
MAX_STOP_TOKEN_IDS = 8

FINISH_NONE, FINISH_LENGTH, FINISH_STOP_EOS, FINISH_STOP_TOKEN, FINISH_ABORT, FINISH_ERROR = range(6)


class TgisConfig(C.Structure):
    _fields_ = [
        ("abi_version", C.c_int32), ("n_layers", C.c_int32), ("hidden", C.c_int32), ("n_q_heads", C.c_int32),
        ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("ffn", C.c_int32), ("vocab", C.c_int32),
        ("rope_theta", C.c_float), ("rms_eps", C.c_float), ("max_model_len", C.c_int32),
        ("max_num_seqs", C.c_int32), ("max_batched_tokens", C.c_int32), ("kv_cache_bytes", C.c_int64),
        ("gpu_mem_fraction", C.c_float), ("device", C.c_int32), ("tp_size", C.c_int32), ("tp_rank", C.c_int32),
        ("use_cuda_graphs", C.c_int32), ("debug_gemm_ref", C.c_int32), ("seed", C.c_uint64),
        ("nccl_id", C.c_uint8 * 128), ("shm_name", C.c_char * 64),
        ("max_loras", C.c_int32), ("max_lora_rank", C.c_int32), ("arch", C.c_int32), ("reserved0", C.c_int32),
    ]


class TgisLayerSpec(C.Structure):
    _fields_ = [
        ("mixer", C.c_int32), ("heads", C.c_int32), ("dim", C.c_int32), ("rot_dim", C.c_int32), ("vdim", C.c_int32),
        ("kv_rank", C.c_int32), ("q_rank", C.c_int32), ("window", C.c_int32), ("rot_dims", C.c_int32),
        ("rot_base", C.c_float), ("scale", C.c_float), ("mlp", C.c_int32), ("experts", C.c_int32), ("top", C.c_int32),
        ("expert_ff", C.c_int32), ("shared_ff", C.c_int32), ("ff", C.c_int32),
        ("kv_heads", C.c_int32), ("softcap", C.c_float), ("qt_coef", C.c_float), ("qt_every", C.c_int32),
        ("mm_heads", C.c_int32), ("mm_dim", C.c_int32), ("mm_vdim", C.c_int32), ("gate_cap", C.c_float),
        ("inner", C.c_int32), ("state", C.c_int32), ("dt_rank", C.c_int32), ("conv", C.c_int32),
        ("decay_rank", C.c_int32), ("reserved", C.c_int32),
        ("kv_from", C.c_int32), ("yarn_factor", C.c_float), ("yarn_original", C.c_float), ("yarn_fast", C.c_float),
        ("yarn_slow", C.c_float), ("groups", C.c_int32), ("norm_groups", C.c_int32), ("gate_rank", C.c_int32),
        ("pool", C.c_int32), ("rot_linear", C.c_float), ("flags", C.c_int32), ("reserved2", C.c_int32),
    ]


class TgisKLatentGeom(C.Structure):
    _fields_ = [
        ("heads", C.c_int32), ("dim", C.c_int32), ("rot_dim", C.c_int32), ("vdim", C.c_int32), ("kv_rank", C.c_int32),
        ("q_rank", C.c_int32), ("window", C.c_int32), ("rot_dims", C.c_int32), ("scale", C.c_float),
    ]


class TgisKCapAttnGeom(C.Structure):
    _fields_ = [
        ("heads", C.c_int32), ("kv_heads", C.c_int32), ("dim", C.c_int32), ("vdim", C.c_int32), ("scale", C.c_float),
        ("softcap", C.c_float), ("qt_coef", C.c_float), ("qt_every", C.c_int32),
    ]


class TgisKSigAttnGeom(C.Structure):
    _fields_ = [
        ("heads", C.c_int32), ("kv_heads", C.c_int32), ("dim", C.c_int32), ("vdim", C.c_int32), ("window", C.c_int32),
        ("rot_dims", C.c_int32), ("scale", C.c_float),
    ]


class TgisKPoolAttnGeom(C.Structure):
    _fields_ = [
        ("heads", C.c_int32), ("kv_heads", C.c_int32), ("dim", C.c_int32), ("vdim", C.c_int32), ("window", C.c_int32),
        ("pool", C.c_int32), ("rot_dims", C.c_int32), ("scale", C.c_float), ("unit_norm", C.c_int32),
    ]


class TgisModelSpec(C.Structure):
    _fields_ = [
        ("n_layers", C.c_int32), ("dtype", C.c_int32), ("embed_scale", C.c_float), ("residual_mult", C.c_float),
        ("norm_eps", C.c_float), ("style", C.c_int32), ("layers", C.POINTER(TgisLayerSpec)),
        ("logit_scale", C.c_float), ("side_dim", C.c_int32),
        ("loop_start", C.c_int32), ("loop_stop", C.c_int32), ("loop_times", C.c_int32), ("reserved", C.c_int32),
    ]


class TgisTraceEntry(C.Structure):
    _fields_ = [
        ("request_id", C.c_char_p), ("tokens", C.POINTER(C.c_int32)), ("n_tokens", C.c_int32), ("n_want", C.c_int32),
        ("want", C.POINTER(C.c_int32)),
    ]


class TgisSamplingParams(C.Structure):
    _fields_ = [
        ("greedy", C.c_int32), ("temperature", C.c_float), ("top_k", C.c_int32), ("top_p", C.c_float),
        ("typical_p", C.c_float), ("repetition_penalty", C.c_float), ("has_length_penalty", C.c_int32),
        ("lp_start_index", C.c_uint32), ("lp_decay_factor", C.c_float), ("eos_token_id", C.c_int32),
        ("min_tokens", C.c_int32), ("max_tokens", C.c_int32), ("num_logprobs", C.c_int32),
        ("prompt_logprobs", C.c_int32), ("has_seed", C.c_int32), ("seed", C.c_uint64),
        ("n_stop_token_ids", C.c_int32), ("stop_token_ids", C.c_int32 * MAX_STOP_TOKEN_IDS),
        ("guided", C.c_int32), ("lora_slot", C.c_int32),
    ]


class TgisStepOutput(C.Structure):
    _fields_ = [
        ("request_id", C.c_char * MAX_REQUEST_ID), ("n_new_tokens", C.c_int32), ("token_id", C.c_int32),
        ("logprob", C.c_float), ("rank", C.c_int32), ("n_topn", C.c_int32), ("topn_ids", C.c_int32 * MAX_TOPN),
        ("topn_logprobs", C.c_float * MAX_TOPN), ("finish_reason", C.c_int32), ("stop_token_id", C.c_int32),
        ("n_prompt_tokens", C.c_int32), ("n_output_tokens", C.c_int32), ("ts_arrival", C.c_double),
        ("ts_first_scheduled", C.c_double), ("ts_first_token", C.c_double), ("ts_last_token", C.c_double),
        ("prompt_pos", C.c_int32), ("reserved", C.c_int32),
    ]


class TgisStatus(C.Structure):
    _fields_ = [
        ("errored", C.c_int32), ("is_running", C.c_int32), ("n_running", C.c_int32), ("n_waiting", C.c_int32),
        ("free_blocks", C.c_int32), ("total_blocks", C.c_int32), ("steps", C.c_int64),
        ("tokens_generated", C.c_int64), ("kernel_launches", C.c_int64), ("gpu_busy_ms", C.c_double),
        ("gpu_decode_ms", C.c_double), ("gpu_mixed_ms", C.c_double), ("decode_steps", C.c_int64),
        ("decode_tokens", C.c_int64), ("h2d_bytes", C.c_int64), ("d2h_bytes", C.c_int64), ("gemm_ms", C.c_double),
        ("gemm_bytes", C.c_double), ("gemm_calls", C.c_int64), ("graph_launches", C.c_int64),
        ("exchange_ms", C.c_double), ("exchange_calls", C.c_int64), ("preemptions", C.c_int64),
    ]


# Every symbol include/tgis_engine.h and include/tgis_kernels.h declare (tests/test_abi_cpu.py checks the export list)
ENGINE_SYMBOLS = [
    "tgis_last_error", "tgis_abi_version", "tgis_engine_create", "tgis_engine_create_spec", "tgis_engine_trace_step", "tgis_engine_load_weight", "tgis_engine_start",
    "tgis_engine_add_request", "tgis_engine_abort", "tgis_engine_set_mask_provider", "tgis_engine_load_adapter_weight", "tgis_engine_clear_adapter", "tgis_engine_poll", "tgis_engine_status",
    "tgis_engine_max_model_len", "tgis_engine_set_profiling", "tgis_nccl_unique_id", "tgis_engine_worker_run", "tgis_engine_shutdown", "tgis_engine_destroy", "tgis_engine_run_until_idle",
]
KERNEL_SYMBOLS = [
    "tgis_k_last_error", "tgis_k_gemm_timeline", "tgis_k_step_timeline_enable", "tgis_k_step_timeline_read", "tgis_k_gemm", "tgis_k_rmsnorm", "tgis_k_opt_layernorm", "tgis_k_opt_bias_act", "tgis_k_opt_embed", "tgis_k_silu_mul", "tgis_k_rope_kv", "tgis_k_gemm_rope", "tgis_k_gemm_norm_chain", "tgis_k_attention",
    "tgis_k_attention_bench", "tgis_k_decode_items", "tgis_k_gemm_plan", "tgis_k_gemm_unit_rows",
    "tgis_k_sampler", "tgis_k_sampler_ex", "tgis_k_sampler_masked", "tgis_k_lora", "tgis_k_lora_bench", "tgis_k_silu_mul_interleaved", "tgis_k_gemm_any", "tgis_k_rmsnorm_f32", "tgis_k_resid_tail", "tgis_k_latent_prep", "tgis_k_latent_q_rope", "tgis_k_latent_attn", "tgis_k_moe_route", "tgis_k_moe_align", "tgis_k_capattn_prep", "tgis_k_capattn", "tgis_k_sigattn_prep", "tgis_k_sigattn", "tgis_k_poolattn_prep", "tgis_k_poolattn", "tgis_k_delta_scan", "tgis_k_ssd_scan", "tgis_k_token_shift", "tgis_k_short_conv", "tgis_k_selective_scan", "tgis_k_outer_scan", "tgis_k_head_norm_gate", "tgis_k_resid_tail_pair", "tgis_k_sizeof_sample_row", "tgis_k_sizeof_sample_out", "tgis_k_kv_block",
]

_LIB: C.CDLL | None = None


def library_path() -> Path:
    override = os.environ.get("TGIS_ENGINE_LIB")   # experiments: an alternative build of the same sources
    if override:
        return Path(override)
    return Path(__file__).resolve().parent.parent / "lib" / "libtgis_engine.so"


def load_library() -> C.CDLL:
    """Load (building first if needed) the native engine.  Raises if neither is possible — no fallback."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not os.environ.get("TGIS_ENGINE_LIB"):
        # build() is a digest compare when the library is current; it rebuilds after ANY source/header edit, so tests
        # and benchmarks can never validate a stale .so.  Without nvcc (a deployment box) an existing library is used.
        from vllm_tgis_adapter_b200.csrc.build import build, have_nvcc

        if have_nvcc() or not path.exists():
            build(force=bool(os.environ.get("TGIS_FORCE_BUILD")))
    if not path.exists():
        raise RuntimeError(f"{path} is missing and could not be built: the TGIS B200 engine has no fallback path")
    lib = C.CDLL(str(path))
    vp, i32, i64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float
    lib.tgis_last_error.restype = C.c_char_p
    lib.tgis_k_last_error.restype = C.c_char_p
    lib.tgis_engine_create.argtypes = [C.POINTER(TgisConfig), C.POINTER(vp)]
    lib.tgis_engine_create_spec.argtypes = [C.POINTER(TgisConfig), C.POINTER(TgisModelSpec), C.POINTER(vp)]
    lib.tgis_engine_trace_step.argtypes = [vp, C.POINTER(TgisTraceEntry), i32, C.POINTER(C.c_char_p), i32, C.POINTER(f32)]
    lib.tgis_engine_load_weight.argtypes = [vp, C.c_char_p, vp, i64, i64, i32]
    lib.tgis_engine_start.argtypes = [vp]
    lib.tgis_engine_add_request.argtypes = [vp, C.c_char_p, C.POINTER(i32), i32, C.POINTER(TgisSamplingParams)]
    lib.tgis_engine_abort.argtypes = [vp, C.c_char_p]
    lib.tgis_engine_set_mask_provider.argtypes = [vp, vp, vp]
    lib.tgis_engine_load_adapter_weight.argtypes = [vp, i32, C.c_char_p, vp, i64, i64]
    lib.tgis_engine_clear_adapter.argtypes = [vp, i32]
    lib.tgis_engine_poll.argtypes = [vp, C.POINTER(TgisStepOutput), i32, i32]
    lib.tgis_engine_status.argtypes = [vp, C.POINTER(TgisStatus)]
    lib.tgis_engine_max_model_len.argtypes = [vp]
    lib.tgis_engine_set_profiling.argtypes = [vp, i32]
    lib.tgis_nccl_unique_id.argtypes = [C.POINTER(C.c_uint8 * 128)]
    lib.tgis_engine_worker_run.argtypes = [vp]
    lib.tgis_engine_shutdown.argtypes = [vp]
    lib.tgis_engine_destroy.argtypes = [vp]
    lib.tgis_engine_destroy.restype = None
    lib.tgis_engine_run_until_idle.argtypes = [vp]
    lib.tgis_k_gemm.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, i32, C.POINTER(f32), i32]
    lib.tgis_k_rmsnorm.argtypes = [vp, vp, vp, vp, i32, i32, f32]
    lib.tgis_k_gemm_norm_chain.argtypes = [vp, i32, vp, vp, vp, vp, vp, i32, i32, i32, i32, f32, i32, i32, i32,
                                           C.POINTER(f32)]
    lib.tgis_k_silu_mul.argtypes = [vp, vp, i32, i32]
    lib.tgis_k_opt_layernorm.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, f32]
    lib.tgis_k_opt_bias_act.argtypes = [vp, vp, vp, i32, i32, i32]
    lib.tgis_k_opt_embed.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32]
    lib.tgis_k_rope_kv.argtypes = [vp, C.POINTER(i32), C.POINTER(i32), vp, vp, vp, i32, i32, i32]
    lib.tgis_k_attention.argtypes = [vp, vp, vp, C.POINTER(i32), i32, C.POINTER(i32), i32, i32, vp, i32, i32, f32]
    lib.tgis_k_sampler.argtypes = [vp, i32, i32, vp, i32, vp, vp]
    lib.tgis_k_sampler_ex.argtypes = [vp, i32, i32, i32, vp, i32, vp, vp, i32, C.POINTER(f32)]
    lib.tgis_k_lora.argtypes = [vp, i32, vp, vp, vp, i32, i32, i32, i32, vp, i32, i32]
    lib.tgis_k_silu_mul_interleaved.argtypes = [vp, vp, i32, i32]
    lib.tgis_k_lora_bench.argtypes = [vp, i32, vp, vp, vp, i32, i32, i32, vp, i32, i32, i32, C.POINTER(f32), C.POINTER(f32)]
    lib.tgis_k_sampler_masked.argtypes = [vp, i32, i32, i32, vp, i32, vp, vp, vp, i32, C.POINTER(f32)]
    gp = C.POINTER(TgisKLatentGeom)
    lib.tgis_k_gemm_any.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i64, i64, i64, vp, i32, i64,
                                    vp, i32, i32, vp, i32]
    lib.tgis_k_rmsnorm_f32.argtypes = [vp, i32, vp, f32, vp, i32, i32, i32, i32, f32]
    lib.tgis_k_resid_tail.argtypes = [vp, vp, vp, vp, i32, vp, vp, vp, vp, vp, vp, i32, f32, f32, f32, i32, i32]
    lib.tgis_k_latent_prep.argtypes = [vp, i32, gp, vp, vp, f32, vp, vp, vp, vp, vp, i32, vp, i32]
    lib.tgis_k_latent_q_rope.argtypes = [vp, i32, gp, vp, vp, vp, i32]
    lib.tgis_k_latent_attn.argtypes = [vp, vp, i32, C.POINTER(i32), i32, C.POINTER(i32), i32, i32, vp, i32, gp]
    lib.tgis_k_moe_route.argtypes = [vp, i32, vp, i32, i32, vp, vp, vp, i32]
    lib.tgis_k_moe_align.argtypes = [vp, i32, i32, i32, vp, vp, vp]
    cg, ip = C.POINTER(TgisKCapAttnGeom), C.POINTER(i32)
    lib.tgis_k_capattn_prep.argtypes = [vp, i32, i32, i32, i32, cg, vp, vp, f32, vp, vp, vp, vp, vp, i32, i32]
    lib.tgis_k_capattn.argtypes = [vp, vp, vp, i32, ip, i32, ip, i32, i32, vp, i32, vp, cg]
    sg = C.POINTER(TgisKSigAttnGeom)
    lib.tgis_k_sigattn_prep.argtypes = [vp, i32, i32, i32, i32, sg, vp, vp, vp, vp, vp, vp, i32, i32]
    lib.tgis_k_sigattn.argtypes = [vp, vp, vp, i32, ip, i32, ip, i32, i32, vp, vp, sg]
    pg = C.POINTER(TgisKPoolAttnGeom)
    lib.tgis_k_poolattn_prep.argtypes = [vp, i32, i32, i32, i32, vp, pg, vp, f32, vp, vp, vp, vp, vp, i32, i32]
    lib.tgis_k_poolattn.argtypes = [vp, vp, vp, vp, vp, i32, ip, i32, ip, i32, i32, vp, pg]
    lib.tgis_k_delta_scan.argtypes = [vp, vp, vp, i32, i32, i32, vp, i32, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, i32, ip, i32, vp]
    lib.tgis_k_ssd_scan.argtypes = [vp, vp, vp, i32, i32, i32, vp, i32, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, ip, i32, vp]
    lib.tgis_k_token_shift.argtypes = [vp, i32, vp, i32, vp, vp, vp, vp, i32, i64, i32]
    lib.tgis_k_short_conv.argtypes = [vp, i32, i32, vp, vp, i32, vp, vp, vp, vp, vp, i32, i32]
    lib.tgis_k_selective_scan.argtypes = [vp, vp, i32, vp, i32, i32, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, ip, i32, vp]
    lib.tgis_k_outer_scan.argtypes = [i32, vp, vp, vp, i32, i32, i32, f32, vp, i32, vp, vp, vp, vp, i32, vp, vp, f32, vp, vp, vp,
                                      vp, i32, i32, i32, i32, vp, vp, i32, ip, i32, vp]
    lib.tgis_k_head_norm_gate.argtypes = [vp, i32, i32, i32, vp, vp, i32, i32, f32, vp, i32, i32]
    lib.tgis_k_resid_tail_pair.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, f32, i32, i32]
    _LIB = lib
    return lib


def last_error(lib: C.CDLL) -> str:
    return (lib.tgis_last_error() or b"").decode(errors="replace")
