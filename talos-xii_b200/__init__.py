"""talos_b200: Python host binding of libtalos_b200.so (the C ABI declared in include/*.h).

The directory name is not a Python identifier; load it with `__graft_entry__.load_package()`
(importlib by path, registered as module ``talos_xii_b200``).

Every exported function of the headers is bound by parsing the headers themselves, so the
binding cannot drift from the ABI.  A non-zero status raises `TalosError` carrying
`talos_last_error_string()` -- the reference crate panics in the same situations.  There is
no CPU path: loading the library or creating a context without a CUDA device fails loudly.
"""
import ctypes as C
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
INCLUDE_DIR = os.path.join(os.path.dirname(_HERE), "include")
LIB_PATH = os.path.join(_HERE, "libtalos_b200.so")

OK, ERR_ARG, ERR_SHAPE, ERR_ALLOC, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT, ERR_UNSUPPORTED = range(8)
MODE_FP32, MODE_TF32X3, MODE_TF32 = 0, 1, 2
OP_N, OP_T = 0, 1
ACT_NONE, ACT_RELU, ACT_TANH, ACT_SILU = 0, 1, 2, 3
ROPE_TOKEN, ROPE_HEAD_INDEX = 0, 1
EW = dict(relu=1, tanh=2, silu=3, exp=4, log=5, sin=6, cos=7, sqrt=8, clip=9, neg=10, scale=11, add=20, sub=21, mul=22, div=23)
MODES = {"fp32": MODE_FP32, "tf32x3": MODE_TF32X3, "tf32": MODE_TF32}
ACTS = {None: 0, "none": 0, "relu": 1, "tanh": 2, "silu": 3}


class TalosError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("talos status %d: %s" % (status, message))
        self.status = status


class Epilogue(C.Structure):
    """Mirror of `talos_epilogue` (include/talos_b200.h)."""
    _fields_ = [("bias", C.c_void_p), ("aux_out", C.c_void_p), ("ld_aux_out", C.c_int64), ("aux_in", C.c_void_p),
                ("ld_aux_in", C.c_int64), ("act", C.c_int32), ("dact", C.c_int32), ("beta", C.c_int32)]


_SCALARS = {"int32_t": C.c_int32, "int64_t": C.c_int64, "uint32_t": C.c_uint32, "uint64_t": C.c_uint64, "size_t": C.c_size_t,
            "float": C.c_float, "double": C.c_double, "int": C.c_int, "talos_status": C.c_int32}


def _ctype(decl):
    decl = decl.replace("const", " ").strip()
    stars = decl.count("*")
    base = decl.replace("*", " ").split()
    base = base[0] if base else "void"
    if stars:
        return C.c_void_p
    return _SCALARS[base]


def parse_headers(include_dir=INCLUDE_DIR):
    """Returns {function name: (restype, [argtypes])} for every prototype in include/*.h."""
    protos = {}
    for fn in sorted(os.listdir(include_dir)):
        if not fn.endswith(".h"):
            continue
        text = open(os.path.join(include_dir, fn)).read()
        text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
        text = re.sub(r"//[^\n]*", " ", text)
        text = re.sub(r"typedef\s+struct\s+\w+\s*\{.*?\}\s*\w+\s*;", " ", text, flags=re.S)
        text = re.sub(r"enum\s*\{.*?\}\s*;", " ", text, flags=re.S)
        for m in re.finditer(r"([\w\s\*]+?)\b(talos_\w+)\s*\(([^;{}]*?)\)\s*;", text):
            ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
            if "typedef" in ret:
                continue
            argtypes = []
            if args and args != "void":
                for a in args.split(","):
                    a = a.strip()
                    a = re.sub(r"\b\w+$", "", a).strip() if not a.endswith("*") else a   # drop the parameter name
                    argtypes.append(_ctype(a))
            if "char" in ret:
                restype = C.c_char_p
            else:
                restype = _ctype(ret)
            protos[name] = (restype, argtypes)
    return protos


class _Lib:
    """Attribute access gives a checked callable: status != 0 raises TalosError."""

    def __init__(self):
        if not os.path.exists(LIB_PATH):
            raise ImportError("libtalos_b200.so is not built; run `python talos-xii_b200/build.py` "
                              "(there is no CPU fallback)")
        self.cdll = C.CDLL(LIB_PATH)
        self.protos = parse_headers()
        for name, (restype, argtypes) in self.protos.items():
            f = getattr(self.cdll, name)
            f.restype, f.argtypes = restype, argtypes

    def raw(self, name):
        return getattr(self.cdll, name)

    def __getattr__(self, name):
        protos = self.__dict__.get("protos", {})
        if name not in protos:
            raise AttributeError(name)
        f = getattr(self.cdll, name)
        if protos[name][0] is not C.c_int32 or not name.startswith("talos_") or name in _NOT_STATUS:
            return f

        def checked(*args):
            st = f(*args)
            if st != 0:
                raise TalosError(st, self.cdll.talos_last_error_string().decode())
        checked.__name__ = name
        self.__dict__[name] = checked
        return checked


_NOT_STATUS = {"talos_ctx_tensor_cores_active", "talos_ctx_tensor_cores_state", "talos_comm_peer_exchange_active"}

lib = _Lib()


def ptr(t):
    """Device (or host) address of a torch tensor / numpy array / None as an int for ctypes."""
    if t is None:
        return None
    if hasattr(t, "data_ptr"):
        return t.data_ptr()
    if hasattr(t, "ctypes"):
        return t.ctypes.data
    return int(t)


class Context:
    """One device + one stream (talos_ctx).  `stream` is a raw cudaStream_t value or None."""

    def __init__(self, device=0, stream=None):
        h = C.c_void_p()
        lib.talos_ctx_create(int(device), stream, C.byref(h))
        self.handle = h
        self.device = device

    def synchronize(self):
        lib.talos_ctx_synchronize(self.handle)

    def close(self):
        if self.handle:
            lib.talos_ctx_destroy(self.handle)
            self.handle = None

    @property
    def launches(self):
        return lib.talos_ctx_launch_count(self.handle)

    @property
    def tensor_cores_active(self):
        return bool(lib.talos_ctx_tensor_cores_active(self.handle))

    def timeline_begin(self):
        """Measurement aid: from here every launch through this context is followed by an event (see timeline_end)."""
        lib.talos_ctx_timeline_begin(self.handle)

    def timeline_end(self, capacity=512):
        """Returns [(launch name, microseconds since the previous mark)] for the launches since timeline_begin."""
        n = C.c_int32(); us = (C.c_float * capacity)(); stride = 32
        names = C.create_string_buffer(capacity * stride)
        lib.talos_ctx_timeline_end(self.handle, capacity, C.byref(n), us, names, stride)
        k = min(n.value, capacity)
        return [(names.raw[i * stride:(i + 1) * stride].split(b"\0", 1)[0].decode(), float(us[i])) for i in range(k)]

    @property
    def tensor_cores_state(self):
        """1: in use; 0: not probed yet; -1: the start-up self-check failed and the fp32 kernel serves every mode."""
        return int(lib.talos_ctx_tensor_cores_state(self.handle))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def torch_context(device=0):
    """A Context on torch's current stream for `device`, so torch allocations and copies order
    with the library's kernels (torch is used for device memory and streams only)."""
    import torch
    return Context(device, torch.cuda.current_stream(device).cuda_stream)


# ---------------------------------------------------------------------------------------------
# PPO trainer (include/talos_b200_ppo.h)


class PpoConfig(C.Structure):
    """Mirror of `talos_ppo_config`; defaults are the reference's constants (src/ppo.rs:17-21, :509-511, :567)."""
    _fields_ = [("obs_dim", C.c_int32), ("hidden", C.c_int32), ("n_actions", C.c_int32), ("minibatch", C.c_int32),
                ("mode", C.c_int32), ("clip", C.c_float), ("c_value", C.c_float), ("c_entropy", C.c_float), ("lr", C.c_float),
                ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float)]

    def __init__(self, obs_dim, hidden, n_actions, minibatch, mode=MODE_TF32X3, clip=0.2, c_value=0.5, c_entropy=0.01,
                 lr=3e-4, beta1=0.9, beta2=0.999, eps=1e-8):
        super().__init__(obs_dim, hidden, n_actions, minibatch, mode, clip, c_value, c_entropy, lr, beta1, beta2, eps)


class Comm:
    """NCCL communicator of one rank (talos_comm).  `unique_id()` on rank 0, ship the bytes, then Comm(ctx, id, n, r)."""

    @staticmethod
    def unique_id():
        buf = (C.c_uint8 * 128)()
        lib.talos_comm_unique_id(buf)
        return bytes(buf)

    def __init__(self, ctx, uid, nranks, rank):
        h = C.c_void_p()
        buf = (C.c_uint8 * 128).from_buffer_copy(uid)
        lib.talos_comm_init(ctx.handle, buf, nranks, rank, C.byref(h))
        self.handle, self.ctx, self.nranks, self.rank = h, ctx, nranks, rank

    @property
    def peer_exchange_active(self):
        """True when the ranks have mapped each other's exchange areas (gradient exchange + Adam as one kernel over
        NVLink peer memory); False when the NCCL all-reduce serves."""
        return bool(lib.talos_comm_peer_exchange_active(self.handle))

    def allreduce_sum(self, dev_ptr, n):
        lib.talos_comm_allreduce_sum(self.handle, dev_ptr, n)

    def close(self):
        if self.handle:
            lib.talos_comm_destroy(self.handle)
            self.handle = None


class PPOTrainer:
    """Host mirror of the optimisation half of `PPO` (src/ppo.rs:555-770) for the MLP actor-critic."""
    NAMES = ["w1", "b1", "w2", "b2", "wp", "bp", "wv", "bv"]

    def __init__(self, ctx, cfg, comm=None):
        h = C.c_void_p()
        lib.talos_ppo_create(ctx.handle, C.byref(cfg), C.byref(h))
        self.handle, self.ctx, self.cfg, self.comm = h, ctx, cfg, comm
        n = C.c_int64()
        lib.talos_ppo_param_count(h, C.byref(n))
        self.n_params = n.value

    def _shapes(self):
        c = self.cfg
        return [(c.obs_dim, c.hidden), (c.hidden,), (c.hidden, c.hidden), (c.hidden,), (c.hidden, c.n_actions), (c.n_actions,),
                (c.hidden, 1), (1,)]

    def set_params(self, params):
        """`params`: dict name -> array in the canonical order, or one flat fp32 array."""
        import numpy as np
        if isinstance(params, dict):
            flat = np.concatenate([np.asarray(params[k], dtype=np.float32).ravel() for k in self.NAMES])
        else:
            flat = np.ascontiguousarray(params, dtype=np.float32)
        assert flat.size == self.n_params, "parameter count mismatch"
        lib.talos_ppo_set_params_host(self.handle, ptr(flat))

    def get_params(self):
        import numpy as np
        flat = np.empty(self.n_params, dtype=np.float32)
        lib.talos_ppo_get_params_host(self.handle, ptr(flat))
        out, o = {}, 0
        for k, shp in zip(self.NAMES, self._shapes()):
            n = int(np.prod(shp)); out[k] = flat[o:o + n].reshape(shp); o += n
        return out

    def _split(self, flat):
        import numpy as np
        out, o = {}, 0
        for k, shp in zip(self.NAMES, self._shapes()):
            n = int(np.prod(shp)); out[k] = flat[o:o + n].reshape(shp); o += n
        return out

    def get_grads(self):
        """Mean gradient of the last optimizer step (all ranks), as a dict in the canonical order."""
        import numpy as np
        flat = np.empty(self.n_params, dtype=np.float32)
        lib.talos_ppo_get_grads_host(self.handle, ptr(flat))
        return self._split(flat)

    def reset_optimizer(self):
        lib.talos_ppo_reset_optimizer(self.handle)

    def forward(self, obs_dev, n, logits_dev=None, values_dev=None):
        lib.talos_ppo_forward(self.handle, ptr(obs_dev), n, ptr(logits_dev), ptr(values_dev))

    def log_prob(self, obs_dev, actions_dev, n, out_dev):
        lib.talos_ppo_log_prob(self.handle, ptr(obs_dev), ptr(actions_dev), n, ptr(out_dev))

    def step(self, obs, actions, old_logp, adv, ret, n):
        lib.talos_ppo_step(self.handle, self.comm.handle if self.comm else None, ptr(obs), ptr(actions), ptr(old_logp), ptr(adv), ptr(ret), n)

    def update(self, obs, actions, old_logp, adv, ret, N, epochs, kl_stop=0.0, host=False):
        """Runs the epochs x minibatches loops; returns the per-epoch mean approx-KL list.
        host=True takes HOST arrays (numpy / pinned torch) and copies them inside the call."""
        kls = (C.c_float * max(1, epochs))(); run = C.c_int32()
        fn = lib.talos_ppo_update_host if host else lib.talos_ppo_update
        fn(self.handle, self.comm.handle if self.comm else None, ptr(obs), ptr(actions), ptr(old_logp), ptr(adv), ptr(ret), N, epochs,
           kl_stop, kls, C.byref(run))
        return [kls[i] for i in range(run.value)]

    def last_loss(self):
        v = C.c_float()
        lib.talos_ppo_last_loss(self.handle, C.byref(v))
        return v.value

    @property
    def launches_per_step(self):
        return lib.talos_ppo_launches_per_step(self.handle)

    def close(self):
        if self.handle:
            lib.talos_ppo_destroy(self.handle)
            self.handle = None
