"""Host-side mirror of the reference's MoE operator interface on top of the C ABI (include/zc_moe.h).

The reference reaches its MoE layer through C++ members: ``Model::moe(x, layer, tokens, ...)``
(src/engine/model.cpp:431-557) built from ``Metal::linear`` (router), ``Metal::route``,
``Metal::gated_linear`` / ``linear_into`` and the ``moe_sum`` dispatch (include/engine/metal.hpp:101-119).
``Moe`` below exposes the same operations with the same names, argument meaning and error behaviour
(``ValueError`` for the reference's ``std::invalid_argument``, ``IndexError`` for ``std::out_of_range``,
``RuntimeError`` for ``std::runtime_error``), and nothing else: PyTorch only supplies device memory and
streams. There is no CPU path; without the CUDA library or a device the constructor raises.
"""
import ctypes
import os

import numpy as np

from .records import ARITH_FP32, ARITH_REFERENCE, BF16, F16, F32, MoeConfig

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("ZC_MOE_LIB") or os.path.join(_HERE, "libzc_moe.so")      # ZC_MOE_LIB: another build of the library

ZC_OK, ZC_EINVAL, ZC_ERANGE, ZC_EEXEC, ZC_ECANCELLED, ZC_ENOMEM = 0, -1, -2, -3, -4, -5
STATUS_INVALID_ROUTE, STATUS_TIMEOUT, STATUS_RANGE = 1, 2, 4


class Cancelled(RuntimeError):
    """The reference's "generation cancelled" (src/engine/model.cpp:15)."""

EXPORTS = [
    "zc_moe_desc_finalize", "zc_moe_create", "zc_moe_destroy", "zc_moe_last_error", "zc_last_error",
    "zc_moe_load_layer", "zc_moe_set_router_bias", "zc_moe_layer_buffers", "zc_moe_router", "zc_router_logits_noalloc", "zc_moe_route", "zc_moe_permute",
    "zc_moe_combine", "zc_activation_bf16", "zc_moe_decode", "zc_moe_prefill", "zc_moe_forward", "zc_moe_forward_routed", "zc_moe_hc_mix", "zc_moe_forward_hc", "zc_moe_ep_dispatch", "zc_moe_ep_experts", "zc_moe_ep_combine",
    "zc_moe_ep_export", "zc_moe_ep_attach", "zc_moe_ep_layer", "zc_moe_ep_send", "zc_moe_ep_process", "zc_moe_ep_finish", "zc_moe_ep_stack", "zc_moe_ep_stack_eager",
    "zc_moe_forward_host", "zc_moe_forward_host_async", "zc_moe_set_cancel", "zc_moe_stack",
    "zc_moe_stack_host", "zc_moe_set_option", "zc_moe_stack_eager", "zc_moe_profile_begin", "zc_moe_profile_end", "zc_moe_kernel_name",
    "zc_moe_last_routing", "zc_moe_active_counts", "zc_moe_ep_active_counts", "zc_moe_read_device", "zc_moe_status", "zc_moe_wait_selftest", "zc_moe_launch_count", "zc_synth_fill_layer",
]


class Desc(ctypes.Structure):
    """``zc_moe_desc``."""
    _fields_ = [
        ("hidden", ctypes.c_uint32), ("ffn", ctypes.c_uint32), ("experts", ctypes.c_uint32),
        ("top_k", ctypes.c_uint32), ("layers", ctypes.c_uint32), ("group", ctypes.c_uint32),
        ("max_tokens", ctypes.c_uint32), ("first_expert", ctypes.c_uint32),
        ("local_experts", ctypes.c_uint32), ("reserved0", ctypes.c_uint32),
        ("gate_bits", ctypes.c_uint8), ("up_bits", ctypes.c_uint8), ("down_bits", ctypes.c_uint8),
        ("q8_signed", ctypes.c_uint8), ("meta_dtype", ctypes.c_uint8), ("act_dtype", ctypes.c_uint8),
        ("out_dtype", ctypes.c_uint8), ("router_dtype", ctypes.c_uint8), ("has_shared", ctypes.c_uint8),
        ("arith", ctypes.c_uint8),
        ("shared_gate_bits", ctypes.c_uint8), ("shared_up_bits", ctypes.c_uint8), ("shared_down_bits", ctypes.c_uint8), ("reserved", ctypes.c_uint8 * 3),
        ("record_bytes", ctypes.c_uint64), ("record_stride", ctypes.c_uint64),
    ]


_lib = None


def load_library():
    """Loads libzc_moe.so (built by zerocool_b200.build). Raises if it is missing: there is no fallback."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m zerocool_b200.build` (no CPU fallback exists)")
    lib = ctypes.CDLL(LIB_PATH)
    vp, u32, u64, i32 = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int
    lib.zc_moe_desc_finalize.argtypes = [ctypes.POINTER(Desc)]
    lib.zc_moe_create.argtypes = [ctypes.POINTER(Desc), i32, ctypes.POINTER(vp)]
    lib.zc_moe_destroy.argtypes = [vp]
    lib.zc_moe_destroy.restype = None
    lib.zc_moe_last_error.argtypes = [vp]
    lib.zc_moe_last_error.restype = ctypes.c_char_p
    lib.zc_last_error.restype = ctypes.c_char_p
    lib.zc_moe_load_layer.argtypes = [vp, u32, vp, u32, u32, vp, vp, vp]
    lib.zc_moe_set_router_bias.argtypes = [vp, u32, vp]
    lib.zc_moe_layer_buffers.argtypes = [vp, u32, ctypes.POINTER(vp), ctypes.POINTER(vp), ctypes.POINTER(vp), ctypes.POINTER(vp)]
    lib.zc_moe_router.argtypes = [vp, u32, vp, u32, vp, vp]
    lib.zc_router_logits_noalloc.argtypes = [vp, i32, vp, i32, u32, u32, u32, vp, vp]
    lib.zc_moe_route.argtypes = [vp, vp, u32, vp, vp, vp]
    lib.zc_moe_permute.argtypes = [vp, vp, u32, vp, vp, vp]
    lib.zc_moe_combine.argtypes = [vp, vp, vp, vp, vp, vp, u32, vp, vp]
    lib.zc_activation_bf16.argtypes = [vp, u32, vp, vp, vp]
    for name in ("zc_moe_decode", "zc_moe_prefill", "zc_moe_forward"):
        getattr(lib, name).argtypes = [vp, u32, vp, u32, vp, vp]
    lib.zc_moe_forward_routed.argtypes = [vp, u32, vp, u32, vp, vp, vp]
    lib.zc_moe_hc_mix.argtypes = [vp, vp, vp, u32, vp, vp]
    lib.zc_moe_forward_hc.argtypes = [vp, u32, vp, u32, vp, vp, vp, vp]
    lib.zc_moe_ep_dispatch.argtypes = [vp, u32, vp, u32, vp, vp, vp]
    lib.zc_moe_ep_experts.argtypes = [vp, u32, vp, vp, u32, vp, vp]
    lib.zc_moe_ep_combine.argtypes = [vp, u32, vp, u32, vp, vp, vp]
    lib.zc_moe_ep_export.argtypes = [vp, vp, ctypes.POINTER(vp)]
    lib.zc_moe_ep_attach.argtypes = [vp, u32, u32, vp, i32]
    lib.zc_moe_ep_layer.argtypes = [vp, u32, vp, u32, vp, vp]
    lib.zc_moe_ep_send.argtypes = [vp, u32, vp, u32, vp]
    lib.zc_moe_ep_process.argtypes = [vp, u32, vp]
    lib.zc_moe_ep_finish.argtypes = [vp, u32, vp, u32, vp, vp]
    lib.zc_moe_ep_stack.argtypes = [vp, vp, u32, vp, vp]
    lib.zc_moe_ep_stack_eager.argtypes = [vp, vp, u32, vp, vp]
    lib.zc_moe_forward_host.argtypes = [vp, u32, vp, u32, vp, vp]
    lib.zc_moe_forward_host_async.argtypes = [vp, u32, vp, u32, vp, vp]
    lib.zc_moe_set_cancel.argtypes = [vp, vp]
    lib.zc_moe_stack.argtypes = [vp, vp, u32, vp, vp]
    lib.zc_moe_stack_host.argtypes = [vp, vp, u32, vp, vp]
    lib.zc_moe_active_counts.argtypes = [vp, vp]
    lib.zc_moe_ep_active_counts.argtypes = [vp, vp]
    lib.zc_moe_set_option.argtypes = [vp, ctypes.c_char_p, i32]
    lib.zc_moe_stack_eager.argtypes = [vp, vp, u32, vp, vp]
    lib.zc_moe_profile_begin.argtypes = [vp]
    lib.zc_moe_profile_end.argtypes = [vp, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(u64)]
    lib.zc_moe_kernel_name.argtypes = [i32]
    lib.zc_moe_kernel_name.restype = ctypes.c_char_p
    lib.zc_moe_last_routing.argtypes = [vp] + [ctypes.POINTER(vp)] * 5
    lib.zc_moe_read_device.argtypes = [vp, vp, vp, u64]
    lib.zc_moe_status.argtypes = [vp, vp, ctypes.POINTER(u32)]
    lib.zc_moe_wait_selftest.argtypes = [vp, u32, ctypes.POINTER(u32), vp]
    lib.zc_moe_launch_count.argtypes = [vp]
    lib.zc_moe_launch_count.restype = u64
    lib.zc_synth_fill_layer.argtypes = [vp, u32, u64, vp]
    _lib = lib
    return lib


def make_desc(cfg: MoeConfig):
    d = Desc()
    for name, value in cfg.as_dict().items():
        setattr(d, name, int(value))
    return d


def _raise(code, text):
    text = text.decode() if isinstance(text, bytes) else str(text)
    if code == ZC_EINVAL:
        raise ValueError(text)
    if code == ZC_ERANGE:
        raise IndexError(text)
    if code == ZC_ENOMEM:
        raise MemoryError(text)
    if code == ZC_ECANCELLED:
        raise Cancelled(text)
    raise RuntimeError(text)


def _ptr(t):
    """Device or host address of a torch tensor / numpy array / int."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    if isinstance(t, np.ndarray):
        return t.ctypes.data
    return t.data_ptr()


class Moe:
    """One handle = the MoE layers of a model resident in HBM on one device."""

    def __init__(self, cfg: MoeConfig, device=0):
        import torch
        self._torch = torch
        self.lib = load_library()
        cfg.validate()
        self.cfg = cfg
        self.device = torch.device("cuda", device)
        self._h = ctypes.c_void_p()
        desc = make_desc(cfg)
        rc = self.lib.zc_moe_create(ctypes.byref(desc), int(device), ctypes.byref(self._h))
        if rc != ZC_OK:
            _raise(rc, self.lib.zc_last_error())
        self.act_torch = torch.bfloat16 if cfg.act_dtype == BF16 else torch.float32
        self.out_torch = torch.bfloat16 if cfg.out_dtype == BF16 else torch.float32

    # -- lifetime ------------------------------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            self.lib.zc_moe_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc):
        if rc != ZC_OK:
            _raise(rc, self.lib.zc_moe_last_error(self._h))

    def _stream(self):
        return self._torch.cuda.current_stream(self.device).cuda_stream

    # -- weights -------------------------------------------------------------------------------
    def load_layer(self, layer, records=None, first_expert=0, router_w=None, shared_record=None, shared_gate_w=None):
        """records: uint8 [count, record_stride] (numpy or torch, host or device)."""
        count = 0 if records is None else int(records.shape[0])
        keep = [np.ascontiguousarray(a) if isinstance(a, np.ndarray) else a for a in (records, router_w, shared_record, shared_gate_w)]
        self._check(self.lib.zc_moe_load_layer(self._h, layer, _ptr(keep[0]), first_expert, count, _ptr(keep[1]), _ptr(keep[2]), _ptr(keep[3])))

    def set_router_bias(self, layer, bias):
        """bias: fp32 numpy [E] (or None to remove it)."""
        keep = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        self._check(self.lib.zc_moe_set_router_bias(self._h, layer, _ptr(keep)))

    def synth_fill_layer(self, layer, seed):
        self._check(self.lib.zc_synth_fill_layer(self._h, layer, seed, self._stream()))

    def layer_buffers(self, layer):
        ptrs = [ctypes.c_void_p() for _ in range(4)]
        self._check(self.lib.zc_moe_layer_buffers(self._h, layer, *[ctypes.byref(p) for p in ptrs]))
        return dict(records=ptrs[0].value, router_w=ptrs[1].value, shared_record=ptrs[2].value, shared_gate_w=ptrs[3].value)

    def read_device(self, ptr, nbytes):
        """Blocking copy of handle-owned device memory to a numpy uint8 array."""
        out = np.empty(nbytes, np.uint8)
        self._check(self.lib.zc_moe_read_device(self._h, out.ctypes.data, ptr, nbytes))
        return out

    def read_layer_tensor(self, layer, which, nbytes, offset=0):
        """Bytes of a resident tensor (tests of the synthetic generator)."""
        return self.read_device(self.layer_buffers(layer)[which] + offset, nbytes)

    # -- operators (names follow class Metal / Model::moe) ---------------------------------------
    def router(self, layer, x):
        """Metal::linear(router gate, x, tokens, float_output=True): logits [T, E] fp32."""
        torch = self._torch
        tokens = x.shape[0]
        logits = torch.empty((tokens, self.cfg.experts), dtype=torch.float32, device=self.device)
        self._check(self.lib.zc_moe_router(self._h, layer, _ptr(x), tokens, _ptr(logits), self._stream()))
        return logits

    def route(self, logits, tokens=None):
        """Metal::route: (ids int32 [T,K], weights fp32 [T,K])."""
        torch = self._torch
        if tokens is None:
            tokens = logits.shape[0]
        if logits.numel() != tokens * self.cfg.experts:
            raise ValueError("invalid route selection buffers")
        ids = torch.empty((tokens, self.cfg.top_k), dtype=torch.int32, device=self.device)
        weights = torch.empty((tokens, self.cfg.top_k), dtype=torch.float32, device=self.device)
        self._check(self.lib.zc_moe_route(self._h, _ptr(logits), tokens, _ptr(ids), _ptr(weights), self._stream()))
        return ids, weights

    def permute(self, ids):
        """Device-side dispatch lists: (offsets int32 [E+1], perm int32 [T*K])."""
        torch = self._torch
        tokens = ids.shape[0]
        offsets = torch.empty(self.cfg.experts + 1, dtype=torch.int32, device=self.device)
        perm = torch.full((tokens * self.cfg.top_k,), -1, dtype=torch.int32, device=self.device)
        self._check(self.lib.zc_moe_permute(self._h, _ptr(ids), tokens, _ptr(offsets), _ptr(perm), self._stream()))
        return offsets, perm

    def combine(self, expert_out, weights, ids, shared=None, gate_logit=None, out=None):
        """moe_sum on caller tensors: expert_out [T,K,H] fp32, weights [T,K] fp32, ids [T,K] int32, shared [T,H] / gate_logit [T]."""
        torch = self._torch
        tokens = weights.shape[0]
        if out is None:
            out = torch.empty((tokens, self.cfg.hidden), dtype=self.out_torch, device=self.device)
        self._check(self.lib.zc_moe_combine(self._h, _ptr(expert_out), _ptr(weights), _ptr(ids), _ptr(shared), _ptr(gate_logit), tokens,
                                            _ptr(out), self._stream()))
        return out

    def activation_bf16(self, x):
        """(sigmoid, silu) of the reference's BF16-staged activation on an fp32 device tensor."""
        torch = self._torch
        sg, si = torch.empty_like(x), torch.empty_like(x)
        rc = self.lib.zc_activation_bf16(_ptr(x), x.numel(), _ptr(sg), _ptr(si), self._stream())
        if rc != ZC_OK:
            _raise(rc, self.lib.zc_last_error())
        return sg, si

    def _run(self, fn, layer, x, out):
        torch = self._torch
        tokens = x.shape[0]
        if out is None:
            out = torch.empty((tokens, self.cfg.hidden), dtype=self.out_torch, device=self.device)
        self._check(fn(self._h, layer, _ptr(x), tokens, _ptr(out), self._stream()))
        return out

    def moe(self, layer, x, out=None):
        """Model::moe(x, layer, tokens): out [T, H]."""
        return self._run(self.lib.zc_moe_forward, layer, x, out)

    def hc_mix(self, normed, mix):
        """Model::hyper's hc_mix: normed, mix fp32 [T, 4, H] -> the layer input x [T, H] in the activation dtype."""
        torch = self._torch
        tokens = normed.shape[0]
        x = torch.empty((tokens, self.cfg.hidden), dtype=self.act_torch, device=self.device)
        self._check(self.lib.zc_moe_hc_mix(self._h, _ptr(normed), _ptr(mix), tokens, _ptr(x), self._stream()))
        return x

    def moe_hc(self, layer, x, hyper, inject, out=None):
        """Model::moe followed by hc_add in one pass: hyper fp32 [T, 4, H], inject fp32 [T, 4] -> the updated streams."""
        torch = self._torch
        if out is None:
            out = torch.empty_like(hyper)
        self._check(self.lib.zc_moe_forward_hc(self._h, layer, _ptr(x), x.shape[0], _ptr(hyper), _ptr(inject), _ptr(out), self._stream()))
        return out

    def moe_routed(self, layer, x, ids, out=None):
        """Model::moe with a recorded expert selection (ids int32 [T, K] on the device) instead of the top-k search."""
        torch = self._torch
        tokens = x.shape[0]
        if ids.shape != (tokens, self.cfg.top_k) or ids.dtype != torch.int32:
            raise ValueError("invalid route selection buffers")
        if out is None:
            out = torch.empty((tokens, self.cfg.hidden), dtype=self.out_torch, device=self.device)
        self._check(self.lib.zc_moe_forward_routed(self._h, layer, _ptr(x), tokens, _ptr(ids), _ptr(out), self._stream()))
        return out

    def decode(self, layer, x, out=None):
        return self._run(self.lib.zc_moe_decode, layer, x, out)

    def prefill(self, layer, x, out=None):
        return self._run(self.lib.zc_moe_prefill, layer, x, out)

    # -- expert parallelism (device-side pieces; zerocool_b200/ep.py drives the exchange) ---------------
    def ep_dispatch(self, layer, x):
        """-> (rows [T*K, H] act dtype in expert order, row_experts int32 [T*K], offsets numpy int32 [E+1])."""
        torch = self._torch
        tokens = x.shape[0]
        rows = torch.empty((tokens * self.cfg.top_k, self.cfg.hidden), dtype=self.act_torch, device=self.device)
        experts = torch.full((tokens * self.cfg.top_k,), -1, dtype=torch.int32, device=self.device)
        self._check(self.lib.zc_moe_ep_dispatch(self._h, layer, _ptr(x), tokens, _ptr(rows), _ptr(experts), self._stream()))
        return rows, experts, self.last_offsets()

    def last_offsets(self):
        """Host copy (numpy int32 [E + 1]) of the last call's expert offsets: one small device-to-host copy."""
        ptrs = [ctypes.c_void_p() for _ in range(5)]
        self._check(self.lib.zc_moe_last_routing(self._h, *[ctypes.byref(p) for p in ptrs]))
        return self.read_device(ptrs[2].value, (self.cfg.experts + 1) * 4).view(np.int32)

    def ep_experts(self, layer, rows, row_experts):
        torch = self._torch
        n = rows.shape[0]
        y = torch.empty((n, self.cfg.hidden), dtype=torch.float32, device=self.device)
        if n:
            self._check(self.lib.zc_moe_ep_experts(self._h, layer, _ptr(rows), _ptr(row_experts), n, _ptr(y), self._stream()))
        return y

    def ep_combine(self, layer, x, y_sorted, out=None):
        torch = self._torch
        tokens = x.shape[0]
        if out is None:
            out = torch.empty((tokens, self.cfg.hidden), dtype=self.out_torch, device=self.device)
        self._check(self.lib.zc_moe_ep_combine(self._h, layer, _ptr(x), tokens, _ptr(y_sorted), _ptr(out), self._stream()))
        return out

    # -- expert parallelism over peer memory (no collective library, no host value per layer) ------------
    def ep_export(self):
        """-> (64-byte inter-process handle of this rank's window, its device address)."""
        handle = (ctypes.c_uint8 * 64)()
        window = ctypes.c_void_p()
        self._check(self.lib.zc_moe_ep_export(self._h, handle, ctypes.byref(window)))
        return bytes(handle), window.value

    def ep_attach(self, rank, world, handles=None, pointers=None):
        """handles: list of `world` 64-byte handles (ranks in other processes); pointers: list of `world` window
        addresses (ranks in this process)."""
        if pointers is not None:
            table = (ctypes.c_void_p * world)(*[int(p) for p in pointers])
            self._check(self.lib.zc_moe_ep_attach(self._h, rank, world, table, 1))
        else:
            blob = b"".join(handles)
            if len(blob) != 64 * world:
                raise ValueError("one 64-byte handle per rank is needed")
            self._check(self.lib.zc_moe_ep_attach(self._h, rank, world, blob, 0))

    def ep_attach_group(self, dist, group=None):
        """Exchanges the window handles over the (already initialised) process group and attaches; ends with a barrier,
        after which every rank may issue expert-parallel layers."""
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        try:
            handle, error = self.ep_export()[0], None
        except (RuntimeError, ValueError) as exc:
            handle, error = b"\0" * 64, str(exc)
        handles = [None] * world
        dist.all_gather_object(handles, (handle, error), group=group)
        if error is None and all(e is None for _, e in handles):
            try:
                self.ep_attach(rank, world, handles=[h for h, _ in handles])
            except (RuntimeError, ValueError) as exc:
                error = str(exc)
        # every rank learns whether every rank attached (this exchange is also the barrier before the first layer)
        errors = [None] * world
        dist.all_gather_object(errors, error, group=group)
        failed = [f"rank {r}: {e}" for r, e in enumerate(errors) if e is not None] + \
                 [f"rank {r}: {e}" for r, (_, e) in enumerate(handles) if e is not None]
        if failed:
            raise RuntimeError("expert-parallel windows could not be attached: " + "; ".join(sorted(set(failed))))

    def ep_layer(self, layer, x, out=None):
        return self._run(self.lib.zc_moe_ep_layer, layer, x, out)

    def ep_send(self, layer, x):
        self._check(self.lib.zc_moe_ep_send(self._h, layer, _ptr(x), x.shape[0], self._stream()))

    def ep_process(self, layer):
        self._check(self.lib.zc_moe_ep_process(self._h, layer, self._stream()))

    def ep_finish(self, layer, x, out=None):
        return self._run(self.lib.zc_moe_ep_finish, layer, x, out)

    def ep_stack(self, x, out=None, eager=False):
        torch = self._torch
        if out is None:
            out = torch.empty((x.shape[0], self.cfg.hidden), dtype=self.out_torch, device=self.device)
        fn = self.lib.zc_moe_ep_stack_eager if eager else self.lib.zc_moe_ep_stack
        self._check(fn(self._h, _ptr(x), x.shape[0], _ptr(out), self._stream()))
        return out

    def set_cancel(self, flag):
        """flag: numpy int32 array of one element another thread may set to non-zero (None removes it). The caller
        keeps the array alive while it is registered."""
        self._cancel_keep = flag
        self._check(self.lib.zc_moe_set_cancel(self._h, None if flag is None else flag.ctypes.data))

    def moe_host_async(self, layer, x_host, out_host):
        """moe_host without the wait: out_host is valid after the stream has been waited for (status() does)."""
        self._check(self.lib.zc_moe_forward_host_async(self._h, layer, _ptr(x_host), x_host.shape[0], _ptr(out_host), self._stream()))
        return out_host

    def moe_host(self, layer, x_host, out_host):
        """Model::moe for host tensors (pinned numpy/torch CPU memory): copies in, runs, copies out, waits."""
        tokens = x_host.shape[0]
        self._check(self.lib.zc_moe_forward_host(self._h, layer, _ptr(x_host), tokens, _ptr(out_host), self._stream()))
        return out_host

    def stack(self, x, out=None):
        torch = self._torch
        tokens = x.shape[0]
        if out is None:
            out = torch.empty((tokens, self.cfg.hidden), dtype=self.out_torch, device=self.device)
        self._check(self.lib.zc_moe_stack(self._h, _ptr(x), tokens, _ptr(out), self._stream()))
        return out

    def set_option(self, name, value):
        self._check(self.lib.zc_moe_set_option(self._h, name.encode(), int(value)))

    def stack_eager(self, x, out=None):
        torch = self._torch
        if out is None:
            out = torch.empty((x.shape[0], self.cfg.hidden), dtype=self.out_torch, device=self.device)
        self._check(self.lib.zc_moe_stack_eager(self._h, _ptr(x), x.shape[0], _ptr(out), self._stream()))
        return out

    def profile_begin(self):
        self._check(self.lib.zc_moe_profile_begin(self._h))

    def profile_end(self):
        """dict kernel name -> (total ms, launches) since profile_begin."""
        ms = (ctypes.c_double * 16)()
        n = (ctypes.c_uint64 * 16)()
        self._check(self.lib.zc_moe_profile_end(self._h, ms, n))
        out = {}
        for k in range(16):
            name = self.lib.zc_moe_kernel_name(k)
            if name:
                out[name.decode()] = (ms[k], int(n[k]))
        return out

    def stack_host(self, x_host, out_host):
        self._check(self.lib.zc_moe_stack_host(self._h, _ptr(x_host), x_host.shape[0], _ptr(out_host), self._stream()))
        return out_host

    def last_routing(self, tokens):
        """Host copies (numpy) of the last call's ids, weights, offsets, perm and logits."""
        ptrs = [ctypes.c_void_p() for _ in range(5)]
        self._check(self.lib.zc_moe_last_routing(self._h, *[ctypes.byref(p) for p in ptrs]))
        K, E = self.cfg.top_k, self.cfg.experts
        shapes = [((tokens, K), np.int32), ((tokens, K), np.float32), ((E + 1,), np.int32),
                  ((tokens * K,), np.int32), ((tokens, E), np.float32)]
        out = {}
        for name, p, (shape, dtype) in zip(("ids", "weights", "offsets", "perm", "logits"), ptrs, shapes):
            n = int(np.prod(shape)) * 4
            out[name] = self.read_device(p.value, n).view(dtype).reshape(shape)
        return out

    def active_counts(self):
        """Routed experts with work in the latest call of each layer (numpy int32 [layers])."""
        out = np.zeros(self.cfg.layers, np.int32)
        self._check(self.lib.zc_moe_active_counts(self._h, out.ctypes.data))
        return out

    def ep_active_counts(self):
        """Experts of this handle's range that received rows in the latest expert-parallel call of each layer."""
        out = np.zeros(self.cfg.layers, np.int32)
        self._check(self.lib.zc_moe_ep_active_counts(self._h, out.ctypes.data))
        return out

    def status(self):
        """Waits for the current stream and returns (then clears) the device status word."""
        word = ctypes.c_uint32()
        self._check(self.lib.zc_moe_status(self._h, self._stream(), ctypes.byref(word)))
        return word.value

    def wait_selftest(self, polls=2000):
        """Runs the bounded waits of the tensor-core kernels against a barrier nothing arrives on; -> the four report
        words (suspending wait, polling wait, abort flag, TMEM base). ZC_STATUS_TIMEOUT is then set in the status word."""
        report = (ctypes.c_uint32 * 4)()
        self._check(self.lib.zc_moe_wait_selftest(self._h, ctypes.c_uint32(polls), report, self._stream()))
        return list(report)

    def check_status(self):
        """Raises like Model::moe ("invalid router output", src/engine/model.cpp:459)."""
        word = self.status()
        if word & STATUS_INVALID_ROUTE:
            raise RuntimeError("invalid router output")
        return word

    @property
    def launches(self):
        return int(self.lib.zc_moe_launch_count(self._h))


def to_device(array, torch_dtype, device):
    """numpy fp32 values -> torch tensor of the activation dtype on the device."""
    import torch
    return torch.from_numpy(np.ascontiguousarray(array)).to(device=device, dtype=torch_dtype)
