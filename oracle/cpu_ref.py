"""ctypes wrapper of the C++ restatement (oracle/cpu_ref.cpp). TEST INFRASTRUCTURE, not product code."""
import ctypes as C
import os

import numpy as np

import qmlp_oracle as oracle

HERE = os.path.dirname(os.path.abspath(__file__))
_ACT = {"relu": 0, "celu": 1, "sine": 2, "identity": 3}


class _Level(C.Structure):
    _fields_ = [("memory_offset", C.c_int64), ("resolution", C.c_int32), ("hash_grid_size", C.c_int32),
                ("hashed", C.c_int32), ("pad", C.c_int32)]


class _Encoding(C.Structure):
    _fields_ = [("is_grid", C.c_int32), ("start_in", C.c_int32), ("n_in", C.c_int32), ("num_outputs", C.c_int32),
                ("n_levels", C.c_int32), ("n_features", C.c_int32), ("concat", C.c_int32), ("pad", C.c_int32),
                ("box_min", C.c_float * 6), ("box_inv_size", C.c_float * 6), ("levels", C.POINTER(_Level)),
                ("table", C.POINTER(C.c_float))]


class _Layer(C.Structure):
    _fields_ = [("channels_in", C.c_int32), ("channels_out", C.c_int32), ("use_bias", C.c_int32),
                ("activation", C.c_int32), ("weights_start", C.c_int64), ("bias_start", C.c_int64)]


class _Network(C.Structure):
    _fields_ = [("num_inputs", C.c_int32), ("num_outputs", C.c_int32), ("num_encodings", C.c_int32),
                ("num_layers", C.c_int32), ("encodings", C.POINTER(_Encoding)), ("layers", C.POINTER(_Layer)),
                ("params", C.POINTER(C.c_float))]


_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(HERE, "_build", "liboracle.so")
        if not os.path.exists(path):
            import build_oracle
            build_oracle.build()
        _lib = C.CDLL(path)
        _lib.oracle_network_forward.argtypes = [C.POINTER(_Network), C.c_void_p, C.c_int64, C.c_void_p, C.c_int]
        _lib.oracle_network_forward.restype = None
        _lib.oracle_num_threads.restype = C.c_int
        _lib.oracle_network_train_step.argtypes = [C.POINTER(_Network), C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                                   C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                                   C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                                   C.POINTER(C.c_int64), C.c_int, C.c_float, C.c_float, C.c_float, C.c_float,
                                                   C.c_int, C.c_int]
        _lib.oracle_network_train_step.restype = C.c_double
    return _lib


def num_threads() -> int:
    return lib().oracle_num_threads()


class CpuNetwork:
    """Holds the C structs (and the numpy arrays they point into) of one network."""

    def __init__(self, spec: "oracle.NetSpec", params: np.ndarray, tables=()):
        self.spec = spec
        self._params = np.ascontiguousarray(params.astype(np.float32))
        tables = list(tables) + [None] * (len(spec.encodings) - len(tables))
        self._tables = [np.ascontiguousarray(t.astype(np.float32)) if t is not None else None for t in tables]
        self._levels = []
        encs = (_Encoding * len(spec.encodings))()
        for i, e in enumerate(spec.encodings):
            encs[i].is_grid = int(e.id == "HashGrid")
            encs[i].start_in, encs[i].n_in, encs[i].num_outputs = e.start_in, e.n_in, e.num_outputs
            if e.id == "HashGrid":
                if e.n_features > 16:
                    raise ValueError("at most 16 features per level")
                lv = (_Level * len(e.levels))()
                for j, l in enumerate(e.levels):
                    lv[j].memory_offset, lv[j].resolution = l.memory_offset, l.resolution
                    lv[j].hash_grid_size, lv[j].hashed = max(l.hash_grid_size, 1), int(l.hashed)
                self._levels.append(lv)
                encs[i].n_levels, encs[i].n_features = e.n_levels, e.n_features
                encs[i].concat = int(e.combination_mode == "concat")
                for k in range(e.n_in):
                    encs[i].box_min[k] = float(e.box_min[k])
                    encs[i].box_inv_size[k] = float(e.box_inv_size[k])
                encs[i].levels = lv
                encs[i].table = self._tables[i].ctypes.data_as(C.POINTER(C.c_float))
        layers = (_Layer * len(spec.layers))()
        for i, l in enumerate(spec.layers):
            layers[i].channels_in, layers[i].channels_out = l.channels_in, l.channels_out
            if not isinstance(l.activation, str):
                raise ValueError("the C++ CPU restatement handles one activation per layer (benchmark configurations)")
            layers[i].use_bias, layers[i].activation = int(l.use_bias), _ACT[l.activation]
            layers[i].weights_start, layers[i].bias_start = l.weights_start, l.bias_start
        self._encs, self._layers = encs, layers
        self.net = _Network(spec.num_inputs, spec.num_outputs, len(spec.encodings), len(spec.layers), encs, layers,
                            self._params.ctypes.data_as(C.POINTER(C.c_float)))

    def forward(self, x: np.ndarray, threads: int = 0) -> np.ndarray:
        x = np.ascontiguousarray(x.astype(np.float32))
        out = np.empty((x.shape[0], self.spec.num_outputs), dtype=np.float32)
        lib().oracle_network_forward(C.byref(self.net), x.ctypes.data, x.shape[0], out.ctypes.data, threads)
        return out

    # -- training step (forward, L2 loss, backward, weight / bias / table gradients, Adam) ------------------------------
    def _training_state(self):
        if getattr(self, "_train", None) is None:
            ne = len(self.spec.encodings)
            z = lambda a: np.zeros_like(a)
            st = {"gp": z(self._params), "mp": z(self._params), "vp": z(self._params),
                  "gt": [z(t) if t is not None else None for t in self._tables],
                  "mt": [z(t) if t is not None else None for t in self._tables],
                  "vt": [z(t) if t is not None else None for t in self._tables], "step": 0}
            ptrs = lambda arrs: (C.c_void_p * ne)(*[a.ctypes.data if a is not None else None for a in arrs])
            st["gt_p"], st["mt_p"], st["vt_p"] = ptrs(st["gt"]), ptrs(st["mt"]), ptrs(st["vt"])
            st["counts"] = (C.c_int64 * ne)(*[t.size if t is not None else 0 for t in self._tables])
            self._train = st
        return self._train

    @property
    def params(self) -> np.ndarray:
        """The fp32 parameter vector the C side reads and (in train_step) updates in place."""
        return self._params

    @property
    def tables(self):
        return self._tables

    def train_step(self, x: np.ndarray, target: np.ndarray, n_global: int = 0, lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8,
                   update=True, threads: int = 0) -> float:
        """One host training step on (x, target); updates parameters, tables and Adam moments in place and returns the
        sum of squared errors. With update=False the gradients are left in ``gradients()`` instead."""
        st = self._training_state()
        x = np.ascontiguousarray(x.astype(np.float32))
        target = np.ascontiguousarray(target.astype(np.float32))
        assert target.shape == (x.shape[0], self.spec.num_outputs)
        if update:
            st["step"] += 1
        return float(lib().oracle_network_train_step(
            C.byref(self.net), x.ctypes.data, target.ctypes.data, x.shape[0], n_global,
            st["gp"].ctypes.data, st["mp"].ctypes.data, st["vp"].ctypes.data, self._params.size,
            st["gt_p"], st["mt_p"], st["vt_p"], st["counts"], max(st["step"], 1), lr, beta1, beta2, eps, int(update), threads))

    def gradients(self):
        """(network gradient, [table gradient per encoding]) left by train_step(update=False)."""
        st = self._training_state()
        return st["gp"], st["gt"]

    def zero_gradients(self):
        st = self._training_state()
        st["gp"][:] = 0
        for g in st["gt"]:
            if g is not None:
                g[:] = 0
