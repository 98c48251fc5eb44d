"""B200 (sm_100a) engine for the GPT-OSS MoE block: Python binding of the C ABI.

The product is ``libgptoss_moe_b200.so`` (CUDA kernels + ``extern "C"`` layer,
declared in ``include/gptoss_moe_b200.h``).  This module only loads it through
``ctypes`` and wraps the handle in :class:`MoeEngine`, whose methods map one to
one onto the C entry points.  There is no CPU fallback: loading fails loudly
when the library has not been built, and every compute call fails with
``GPTOSS_E_CUDA`` when no sm_100 GPU is present.
"""
from __future__ import annotations

import ctypes
import pathlib

import numpy as np

PKG_DIR = pathlib.Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "libgptoss_moe_b200.so"
HEADER_PATH = PKG_DIR.parent / "include" / "gptoss_moe_b200.h"

GPTOSS_OK = 0
GPTOSS_E_INVALID = -1
GPTOSS_E_CUDA = -2
GPTOSS_E_CAPACITY = -3
GPTOSS_E_DEVICE = -4
GPTOSS_E_STATE = -5
GPTOSS_E_COMM = -6

WEIGHTS_BF16 = 0
WEIGHTS_MXFP4 = 1
GEMM_TCGEN05 = 0
GEMM_SIMT = 1
GEMM_PAIR = 2

STAGES = ("route", "permute", "gate_up", "down", "combine", "dispatch", "return")


class MoeConfig(ctypes.Structure):
    """Mirror of gptoss_moe_config_t."""

    _fields_ = [
        ("hidden_dim", ctypes.c_int),
        ("intermediate_dim", ctypes.c_int),
        ("n_experts", ctypes.c_int),
        ("experts_per_token", ctypes.c_int),
        ("n_layers", ctypes.c_int),
        ("max_tokens", ctypes.c_int),
        ("swiglu_limit", ctypes.c_float),
        ("ep_rank", ctypes.c_int),
        ("ep_size", ctypes.c_int),
        ("weight_format", ctypes.c_int),
        ("device", ctypes.c_int),
    ]


class MoeError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"gptoss_moe error {code}: {text}")
        self.code = code


class ModelConfig(ctypes.Structure):
    """gptoss_model_config_t: the reference's Config / .bin header (run.cpp:26-46)."""
    _fields_ = [("vocab_size", ctypes.c_int), ("hidden_dim", ctypes.c_int),
                ("n_experts", ctypes.c_int), ("experts_per_token", ctypes.c_int),
                ("intermediate_dim", ctypes.c_int), ("n_layers", ctypes.c_int),
                ("head_dim", ctypes.c_int), ("n_attn_heads", ctypes.c_int),
                ("n_kv_heads", ctypes.c_int), ("seq_len", ctypes.c_int),
                ("initial_context_length", ctypes.c_int), ("rope_theta", ctypes.c_float),
                ("rope_scaling_factor", ctypes.c_float), ("sliding_window", ctypes.c_int),
                ("swiglu_limit", ctypes.c_float)]


_lib = None


def load_library() -> ctypes.CDLL:
    """Load the native library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; "
            "g.build()'` (there is no fallback path)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    vp, ip, fp = ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_float)
    c_int, c_char_p = ctypes.c_int, ctypes.c_char_p
    sigs = {
        "gptoss_moe_create": (c_int, [ctypes.POINTER(MoeConfig), ctypes.POINTER(vp)]),
        "gptoss_moe_destroy": (c_int, [vp]),
        "gptoss_moe_last_error": (c_char_p, [vp]),
        "gptoss_moe_load_layer_f32": (c_int, [vp, c_int, vp, vp, vp, vp, vp, vp]),
        "gptoss_moe_load_layer_bf16": (c_int, [vp, c_int, vp, vp, vp, vp, vp, vp, c_int]),
        "gptoss_moe_load_layer_mxfp4": (
            c_int,
            [vp, c_int, vp, vp, vp, vp, vp, vp, vp, vp, c_int],
        ),
        "gptoss_moe_forward": (c_int, [vp, c_int, vp, vp, vp, c_int, vp]),
        "gptoss_moe_forward_host": (c_int, [vp, c_int, vp, vp, vp, c_int]),
        "gptoss_moe_forward_host_submit": (c_int, [vp, c_int, vp, vp, vp, c_int, ip]),
        "gptoss_moe_forward_host_wait": (c_int, [vp, c_int]),
        "gptoss_moe_load_ffn_norm": (c_int, [vp, c_int, vp]),
        "gptoss_moe_route": (c_int, [vp, c_int, vp, vp, c_int, vp]),
        "gptoss_moe_permute": (c_int, [vp, vp, c_int, vp]),
        "gptoss_moe_experts": (c_int, [vp, c_int, vp]),
        "gptoss_moe_combine": (c_int, [vp, vp, c_int, vp]),
        "gptoss_moe_rmsnorm": (c_int, [vp, vp, vp, vp, vp, c_int, vp]),
        "gptoss_moe_get_routing": (c_int, [vp, c_int, vp, vp, vp, vp, vp]),
        "gptoss_moe_get_activations": (c_int, [vp, vp, ctypes.c_size_t]),
        "gptoss_moe_set_option": (c_int, [vp, c_char_p, c_int]),
        "gptoss_moe_launch_count": (ctypes.c_longlong, [vp]),
        "gptoss_moe_device_status": (c_int, [vp]),
        "gptoss_moe_stage_ms": (c_int, [vp, c_int, fp]),
        "gptoss_moe_ep_unique_id": (c_int, [vp]),
        "gptoss_moe_ep_init": (c_int, [vp, vp]),
        "gptoss_moe_ep_transport": (c_int, [vp]),
        "gptoss_moe_ep_init_local": (c_int, [ctypes.POINTER(vp), c_int]),
        "gptoss_moe_forward_part": (c_int, [vp, c_int, c_int, vp, vp, vp, c_int, vp]),
        "gptoss_moe_version": (c_char_p, []),
        "gptoss_moe_permute_static": (c_int, [vp, vp, c_int, c_int, c_int, vp, vp, vp, vp, vp]),
        "gptoss_decode_create": (c_int, [ctypes.POINTER(ModelConfig), c_int, c_int,
                                         ctypes.POINTER(vp)]),
        "gptoss_decode_destroy": (c_int, [vp]),
        "gptoss_decode_last_error": (c_char_p, [vp]),
        "gptoss_decode_load_bin": (c_int, [vp, vp]),
        "gptoss_decode_load_weights": (c_int, [vp, vp]),
        "gptoss_decode_step": (c_int, [vp, vp, vp, c_int, vp, vp]),
        "gptoss_decode_get_logits": (c_int, [vp, c_int, vp]),
        "gptoss_decode_moe": (vp, [vp]),
        "gptoss_decode_device_count": (c_int, []),
        "gptoss_decode_create_ep": (c_int, [ctypes.POINTER(ModelConfig), c_int, c_int, c_int, c_int,
                                            ctypes.POINTER(vp)]),
        "gptoss_decode_set_tensor": (c_int, [vp, c_char_p, c_int, vp, c_int, c_int]),
        "gptoss_decode_set_kv": (c_int, [vp, c_int, c_int, c_int, c_int, c_int, vp, vp]),
        "gptoss_decode_get_kv": (c_int, [vp, c_int, c_int, c_int, c_int, c_int, vp, vp]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def _ptr(obj):
    """Raw address of a torch tensor, numpy array, int or None."""
    if obj is None:
        return None
    if isinstance(obj, int):
        return ctypes.c_void_p(obj)
    if isinstance(obj, np.ndarray):
        if not obj.flags["C_CONTIGUOUS"]:
            raise ValueError("array must be C-contiguous")
        return ctypes.c_void_p(obj.ctypes.data)
    if hasattr(obj, "data_ptr"):
        if not obj.is_contiguous():
            raise ValueError("tensor must be contiguous")
        return ctypes.c_void_p(obj.data_ptr())
    raise TypeError(f"cannot take the address of {type(obj)}")


def permute_static(slot_expert, slot_weight, n_rows, top_k, n_experts, expert_offsets, sorted_row,
                   sorted_weight, row_of, stream=0):
    """gptoss_moe_permute_static: the permutation stage without an engine handle and
    without any allocation (scratch is a fixed array inside the library).  All
    arguments are device buffers owned by the caller."""
    lib = load_library()
    rc = lib.gptoss_moe_permute_static(_ptr(slot_expert), _ptr(slot_weight), n_rows, top_k,
                                       n_experts, _ptr(expert_offsets), _ptr(sorted_row),
                                       _ptr(sorted_weight), _ptr(row_of), ctypes.c_void_p(stream))
    if rc != GPTOSS_OK:
        raise MoeError(rc, lib.gptoss_moe_last_error(None).decode())


class MoeEngine:
    """One engine = one gptoss_moe_t handle.  Method names follow the C ABI."""

    def __init__(
        self,
        hidden_dim,
        intermediate_dim,
        n_experts,
        experts_per_token,
        n_layers=1,
        max_tokens=1024,
        swiglu_limit=7.0,
        ep_rank=0,
        ep_size=1,
        weight_format=WEIGHTS_BF16,
        device=0,
    ):
        self.lib = load_library()
        self.cfg = MoeConfig(
            hidden_dim, intermediate_dim, n_experts, experts_per_token, n_layers, max_tokens,
            swiglu_limit, ep_rank, ep_size, weight_format, device,
        )
        self.handle = ctypes.c_void_p()
        rc = self.lib.gptoss_moe_create(ctypes.byref(self.cfg), ctypes.byref(self.handle))
        if rc != GPTOSS_OK:
            text = self.lib.gptoss_moe_last_error(None).decode()
            self.handle = None
            raise MoeError(rc, text)

    @classmethod
    def borrowed(cls, handle, cfg: "MoeConfig"):
        """The engine inside another object (a decode engine): same methods, not owned."""
        self = cls.__new__(cls)
        self.lib = load_library()
        self.cfg = cfg
        self.handle = handle
        self._borrowed = True
        return self

    # -- plumbing
    def _check(self, rc):
        if rc != GPTOSS_OK:
            raise MoeError(rc, self.lib.gptoss_moe_last_error(self.handle).decode())

    def close(self):
        if getattr(self, "handle", None):
            if not getattr(self, "_borrowed", False):
                self.lib.gptoss_moe_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def local_experts(self):
        return self.cfg.n_experts // max(1, self.cfg.ep_size)

    # -- weights
    def load_layer_f32(self, layer, w_router, b_router, w_mlp1, b_mlp1, w_mlp2, b_mlp2):
        arrs = [np.ascontiguousarray(a, dtype=np.float32)
                for a in (w_router, b_router, w_mlp1, b_mlp1, w_mlp2, b_mlp2)]
        self._check(self.lib.gptoss_moe_load_layer_f32(self.handle, layer, *[_ptr(a) for a in arrs]))

    def load_layer_bf16(self, layer, w_router, b_router, w_mlp1, b_mlp1, w_mlp2, b_mlp2,
                        on_device):
        args = [_ptr(a) for a in (w_router, b_router, w_mlp1, b_mlp1, w_mlp2, b_mlp2)]
        self._check(self.lib.gptoss_moe_load_layer_bf16(self.handle, layer, *args,
                                                        1 if on_device else 0))

    def load_layer_mxfp4(self, layer, w_router_bf16, b_router, w1_blocks, w1_scales, b_mlp1,
                         w2_blocks, w2_scales, b_mlp2, on_device):
        args = [_ptr(a) for a in (w_router_bf16, b_router, w1_blocks, w1_scales, b_mlp1,
                                  w2_blocks, w2_scales, b_mlp2)]
        self._check(self.lib.gptoss_moe_load_layer_mxfp4(self.handle, layer, *args,
                                                         1 if on_device else 0))

    # -- compute
    def forward(self, layer, t, x, pos, n_tokens, stream=0):
        self._check(self.lib.gptoss_moe_forward(self.handle, layer, _ptr(t), _ptr(x), _ptr(pos),
                                                n_tokens, ctypes.c_void_p(stream)))

    def forward_host(self, layer, t_host, x_host, pos_host, n_tokens):
        self._check(self.lib.gptoss_moe_forward_host(self.handle, layer, _ptr(t_host),
                                                     _ptr(x_host), _ptr(pos_host), n_tokens))

    def forward_host_submit(self, layer, t_host, x_host, pos_host, n_tokens) -> int:
        ticket = ctypes.c_int()
        self._check(self.lib.gptoss_moe_forward_host_submit(
            self.handle, layer, _ptr(t_host), _ptr(x_host), _ptr(pos_host), n_tokens,
            ctypes.byref(ticket)))
        return int(ticket.value)

    def load_ffn_norm(self, layer, scale):
        scale = np.ascontiguousarray(scale, dtype=np.float32)
        self._check(self.lib.gptoss_moe_load_ffn_norm(self.handle, layer, _ptr(scale)))

    def forward_host_wait(self, ticket: int):
        self._check(self.lib.gptoss_moe_forward_host_wait(self.handle, ticket))

    def route(self, layer, t, pos, n_tokens, stream=0):
        self._check(self.lib.gptoss_moe_route(self.handle, layer, _ptr(t), _ptr(pos), n_tokens,
                                              ctypes.c_void_p(stream)))

    def permute(self, t, n_tokens, stream=0):
        self._check(self.lib.gptoss_moe_permute(self.handle, _ptr(t), n_tokens,
                                                ctypes.c_void_p(stream)))

    def experts(self, layer, stream=0):
        self._check(self.lib.gptoss_moe_experts(self.handle, layer, ctypes.c_void_p(stream)))

    def combine(self, x, n_tokens, stream=0):
        self._check(self.lib.gptoss_moe_combine(self.handle, _ptr(x), n_tokens,
                                                ctypes.c_void_p(stream)))

    def rmsnorm(self, out, x, w_dev, pos, n_tokens, stream=0):
        self._check(self.lib.gptoss_moe_rmsnorm(self.handle, _ptr(out), _ptr(x), _ptr(w_dev),
                                                _ptr(pos), n_tokens, ctypes.c_void_p(stream)))

    # -- taps
    def get_routing(self, n_tokens, want_logits=False):
        K, El, E = self.cfg.experts_per_token, self.local_experts, self.cfg.n_experts
        topk_i = np.empty((n_tokens, K), dtype=np.int32)
        topk_v = np.empty((n_tokens, K), dtype=np.float32)
        offsets = np.empty((El + 1,), dtype=np.int32)
        # under expert parallelism the owner's sorted order holds rows of every rank's batch,
        # whatever this rank's own n_tokens is: size for the engine's capacity
        rows_cap = self.cfg.max_tokens * max(1, self.cfg.ep_size) if self.cfg.ep_size > 1 else n_tokens
        sorted_token = np.full((max(1, rows_cap * K),), -1, dtype=np.int32)
        logits = np.empty((n_tokens, E), dtype=np.float32) if want_logits else None
        self._check(self.lib.gptoss_moe_get_routing(self.handle, n_tokens, _ptr(topk_i),
                                                    _ptr(topk_v), _ptr(offsets),
                                                    _ptr(sorted_token), _ptr(logits)))
        out = {"topk_i": topk_i, "topk_v": topk_v, "expert_offsets": offsets,
               "sorted_token": sorted_token[: int(offsets[-1])]}
        if want_logits:
            out["logits"] = logits
        return out

    def get_activations(self, n_rows):
        buf = np.empty((n_rows, self.cfg.intermediate_dim), dtype=np.uint16)
        self._check(self.lib.gptoss_moe_get_activations(self.handle, _ptr(buf), buf.nbytes))
        return buf

    def set_option(self, name, value):
        self._check(self.lib.gptoss_moe_set_option(self.handle, name.encode(), int(value)))

    def launch_count(self):
        return int(self.lib.gptoss_moe_launch_count(self.handle))

    def device_status(self):
        return int(self.lib.gptoss_moe_device_status(self.handle))

    def stage_ms(self, stage):
        ms = ctypes.c_float()
        idx = STAGES.index(stage) if isinstance(stage, str) else stage
        self._check(self.lib.gptoss_moe_stage_ms(self.handle, idx, ctypes.byref(ms)))
        return float(ms.value)

    # -- expert parallelism
    @staticmethod
    def ep_unique_id():
        lib = load_library()
        buf = (ctypes.c_ubyte * 128)()
        rc = lib.gptoss_moe_ep_unique_id(ctypes.cast(buf, ctypes.c_void_p))
        if rc != GPTOSS_OK:
            raise MoeError(rc, "gptoss_moe_ep_unique_id failed")
        return bytes(buf)

    def ep_init(self, unique_id: bytes):
        buf = (ctypes.c_ubyte * 128).from_buffer_copy(unique_id)
        self._check(self.lib.gptoss_moe_ep_init(self.handle, ctypes.cast(buf, ctypes.c_void_p)))

    @staticmethod
    def ep_init_local(engines):
        """gptoss_moe_ep_init_local: engines[r] was created with ep_rank r, ep_size len(engines);
        all of them live in this process."""
        lib = load_library()
        arr = (ctypes.c_void_p * len(engines))(*[e.handle for e in engines])
        rc = lib.gptoss_moe_ep_init_local(arr, len(engines))
        if rc != GPTOSS_OK:
            text = lib.gptoss_moe_last_error(engines[0].handle).decode()
            for e in engines:
                t2 = lib.gptoss_moe_last_error(e.handle).decode()
                if t2:
                    text = t2
            raise MoeError(rc, text or lib.gptoss_moe_last_error(None).decode())

    def forward_part(self, layer, part, t, x, pos, n_tokens, stream=0):
        self._check(self.lib.gptoss_moe_forward_part(self.handle, layer, part, _ptr(t), _ptr(x),
                                                     _ptr(pos), n_tokens, ctypes.c_void_p(stream)))

    @property
    def ep_transport(self) -> int:
        """0 = NCCL send/recv, 1 = peer memory, -1 before ep_init."""
        return int(self.lib.gptoss_moe_ep_transport(self.handle))


class DecodeEngine:
    """Mirror of include/gptoss_decode_b200.h: one greedy decode step for a batch of
    sequences (row i owns KV-cache slot i)."""

    def __init__(self, cfg: dict, max_batch: int, device: int = 0, ep_rank: int = 0,
                 ep_size: int = 1):
        self.lib = load_library()
        self.cfg = dict(cfg)
        self.max_batch = max_batch
        c = ModelConfig(**cfg)
        h = ctypes.c_void_p()
        rc = self.lib.gptoss_decode_create_ep(ctypes.byref(c), max_batch, device, ep_rank, ep_size,
                                              ctypes.byref(h))
        if rc != 0:
            raise MoeError(rc, (self.lib.gptoss_decode_last_error(None) or b"").decode())
        self.handle = h

    def _check(self, rc):
        if rc != 0:
            raise MoeError(rc, (self.lib.gptoss_decode_last_error(self.handle) or b"").decode())

    def load_bin(self, image: np.ndarray):
        """image: the whole .bin file as a uint8/float32 array (e.g. np.memmap); tensors
        start 60 bytes in."""
        raw = image.view(np.uint8).reshape(-1)
        first = raw[60:]
        self._check(self.lib.gptoss_decode_load_bin(self.handle,
                                                    ctypes.c_void_p(first.ctypes.data)))

    def set_tensor(self, name: str, layer: int, src):
        """src: float32 numpy array (host) or a CUDA torch tensor (bf16 weights, fp32 others)."""
        on_device = hasattr(src, "data_ptr")
        is_bf16 = on_device and str(src.dtype) == "torch.bfloat16"
        self._check(self.lib.gptoss_decode_set_tensor(self.handle, name.encode(), layer, _ptr(src),
                                                      int(on_device), int(is_bf16)))

    def set_kv(self, layer: int, row0: int, pos0: int, k, v):
        """k, v: CUDA bf16 tensors [rows, positions, n_kv_heads * head_dim]."""
        self._check(self.lib.gptoss_decode_set_kv(self.handle, layer, row0, k.shape[0], pos0,
                                                  k.shape[1], _ptr(k), _ptr(v)))

    def get_kv(self, layer: int, row0: int, pos0: int, k, v):
        """Fills the CUDA bf16 tensors k, v [rows, positions, n_kv_heads * head_dim]."""
        self._check(self.lib.gptoss_decode_get_kv(self.handle, layer, row0, k.shape[0], pos0,
                                                  k.shape[1], _ptr(k), _ptr(v)))

    def moe(self, ep_rank: int = 0, ep_size: int = 1, device: int = 0) -> "MoeEngine":
        """The MoE engine inside, with MoeEngine's methods (weights, options, timers, EP)."""
        c = self.cfg
        cfg = MoeConfig(c["hidden_dim"], c["intermediate_dim"], c["n_experts"],
                        c["experts_per_token"], c["n_layers"], self.max_batch, c["swiglu_limit"],
                        ep_rank, ep_size, WEIGHTS_BF16, device)
        return MoeEngine.borrowed(ctypes.c_void_p(self.lib.gptoss_decode_moe(self.handle)), cfg)

    def step(self, tokens, pos, stream: int = 0):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        pos = np.ascontiguousarray(pos, dtype=np.int32)
        nxt = np.empty(tokens.shape[0], dtype=np.int32)
        self._check(self.lib.gptoss_decode_step(self.handle, _ptr(tokens), _ptr(pos),
                                                tokens.shape[0], _ptr(nxt),
                                                ctypes.c_void_p(stream)))
        return nxt

    def logits(self, row: int) -> np.ndarray:
        out = np.empty(self.cfg["vocab_size"], dtype=np.float32)
        self._check(self.lib.gptoss_decode_get_logits(self.handle, row, _ptr(out)))
        return out

    def close(self):
        if getattr(self, "handle", None):
            self.lib.gptoss_decode_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass
