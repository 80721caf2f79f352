"""ctypes binding of libonn_b200_host.so (include/onn_b200_host.h): the C++ host mirror of
OpenNN's NeuralNetwork / Transformer / CrossEntropyError3d / AdaptiveMomentEstimation.

Python holds no compute: it hands raw pointers (torch tensors' device memory, or pinned host
memory) and sizes across the C ABI.  There is no fallback path.
"""

from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import capi

HOST_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libonn_b200_host.so")

TRANSFORMER, DECODER_ONLY = 0, 1

HOST_EXPORTS = [
    "onn_trainer_last_error", "onn_trainer_create", "onn_trainer_destroy", "onn_trainer_parameters_number",
    "onn_trainer_layers_number", "onn_trainer_layer_info", "onn_trainer_set_parameters", "onn_trainer_get_parameters",
    "onn_trainer_get_gradients", "onn_trainer_set_learning_rate", "onn_trainer_set_iteration", "onn_trainer_set_dp",
    "onn_trainer_step_device", "onn_trainer_step_host", "onn_trainer_step_host_i32", "onn_trainer_forward", "onn_trainer_get_layer_output",
    "onn_trainer_synchronize", "onn_trainer_parameters_ready", "onn_trainer_exchange_segments", "onn_trainer_trace_phases", "onn_trainer_last_step_phases", "onn_trainer_stream", "onn_trainer_set_graph_capture", "onn_trainer_set_dp_options",
    "onn_trainer_greedy_decode", "onn_trainer_greedy_decode_cached",
    "onn_classifier_last_error", "onn_classifier_create", "onn_classifier_destroy", "onn_classifier_parameters_number",
    "onn_classifier_layers_number", "onn_classifier_layer_info", "onn_classifier_set_parameters", "onn_classifier_get_parameters",
    "onn_classifier_get_gradients", "onn_classifier_set_learning_rate", "onn_classifier_forward", "onn_classifier_step_device",
    "onn_classifier_get_layer_output", "onn_classifier_layer_output_size", "onn_classifier_set_dp",
]

_host = None


def host_lib():
    global _host
    if _host is None:
        capi.lib()      # the kernel library first (RTLD_GLOBAL), the host mirror links against it
        if not os.path.exists(HOST_LIB_PATH):
            raise capi.OnnError(f"{HOST_LIB_PATH} is missing: run `python -m opennn_b200._build`")
        L = C.CDLL(HOST_LIB_PATH)
        L.onn_trainer_last_error.restype = C.c_char_p
        L.onn_trainer_parameters_number.restype = C.c_int64
        L.onn_trainer_destroy.restype = None
        L.onn_trainer_stream.restype = C.c_void_p
        L.onn_classifier_last_error.restype = C.c_char_p
        L.onn_classifier_parameters_number.restype = C.c_int64
        L.onn_classifier_layer_output_size.restype = C.c_int64
        L.onn_classifier_destroy.restype = None
        _host = L
    return _host


def _check(status, what):
    if status != 0:
        raise capi.OnnError(f"{what}: {host_lib().onn_trainer_last_error().decode()} ({status})")


def _f32_ptr(array):
    return array.ctypes.data_as(C.c_void_p)


class Trainer:
    """One network + CrossEntropyError3d + Adam on the current CUDA device."""

    def __init__(self, kind, S_in, S_dec, V_in, V_out, E, H, F, L, micro_batch):
        self.kind, self.S_in, self.S_dec, self.V_out, self.micro_batch = kind, S_in, S_dec, V_out, micro_batch
        self._handle = C.c_void_p()
        i64 = C.c_int64
        _check(host_lib().onn_trainer_create(C.byref(self._handle), int(kind), i64(S_in), i64(S_dec), i64(V_in), i64(V_out),
                                             i64(E), i64(H), i64(F), i64(L), i64(micro_batch)), "onn_trainer_create")
        self.parameters_number = int(host_lib().onn_trainer_parameters_number(self._handle))
        self.layers_number = int(host_lib().onn_trainer_layers_number(self._handle))

    def close(self):
        if self._handle:
            host_lib().onn_trainer_destroy(self._handle)
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def layer_info(self, i):
        name, label = C.create_string_buffer(128), C.create_string_buffer(128)
        params, out_size = C.c_int64(), C.c_int64()
        _check(host_lib().onn_trainer_layer_info(self._handle, int(i), name, label, 128, C.byref(params), C.byref(out_size)), "layer_info")
        return name.value.decode(), label.value.decode(), params.value, out_size.value

    def set_parameters(self, host_array):
        a = np.ascontiguousarray(host_array, dtype=np.float32)
        assert a.size == self.parameters_number
        _check(host_lib().onn_trainer_set_parameters(self._handle, _f32_ptr(a)), "set_parameters")

    def get_parameters(self):
        a = np.empty(self.parameters_number, dtype=np.float32)
        _check(host_lib().onn_trainer_get_parameters(self._handle, _f32_ptr(a)), "get_parameters")
        return a

    def get_gradients(self):
        a = np.empty(self.parameters_number, dtype=np.float32)
        _check(host_lib().onn_trainer_get_gradients(self._handle, _f32_ptr(a)), "get_gradients")
        return a

    def set_learning_rate(self, lr):
        _check(host_lib().onn_trainer_set_learning_rate(self._handle, C.c_float(lr)), "set_learning_rate")

    def set_graph_capture(self, enabled):
        """CUDA-graph replay of the micro-batches (on by default); results do not depend on it."""
        _check(host_lib().onn_trainer_set_graph_capture(self._handle, int(bool(enabled))), "set_graph_capture")

    def set_dp(self, comm_handle, world):
        _check(host_lib().onn_trainer_set_dp(self._handle, comm_handle, int(world)), "set_dp")

    def set_dp_options(self, sharded_update=True, carve_sms=0, carve_launches=4, bucket_floats=0):
        """Before set_dp.  sharded_update: reduce-scatter the gradient buckets, clip + Adam on this rank's 1/world of
        the arena, all-gather the parameters (False: all-reduce and the whole update on every rank).  carve_sms: SMs
        the persistent kernels leave free for NCCL during the carve_launches launches that follow a bucket.
        bucket_floats: size of a gradient bucket (0 = the default, 64 MiB)."""
        _check(host_lib().onn_trainer_set_dp_options(self._handle, int(bool(sharded_update)), int(carve_sms), int(carve_launches),
                                                     C.c_int64(int(bucket_floats))), "set_dp_options")

    def step_device(self, dec_ids, enc_ids, targets, update=True, want_statistics=True):
        """dec_ids / enc_ids / targets: torch CUDA float tensors [batch, S].  Returns
        (error, accuracy, active tokens, gradient norm) or None."""
        stats = (C.c_float * 4)()
        batch = dec_ids.shape[0]
        _check(host_lib().onn_trainer_step_device(self._handle, capi.ptr(dec_ids), capi.ptr(enc_ids), capi.ptr(targets),
                                                  C.c_int64(batch), int(update), stats if want_statistics else None), "step_device")
        return tuple(stats) if want_statistics else None

    def step_host(self, dec_ids, enc_ids, targets, update=True, want_statistics=True):
        """Same with host memory: torch CPU tensors (pinned for full copy speed) or numpy arrays."""
        stats = (C.c_float * 4)()

        def host_ptr(x):
            if x is None:
                return C.c_void_p(0)
            return C.c_void_p(x.data_ptr()) if hasattr(x, "data_ptr") else _f32_ptr(x)

        batch = dec_ids.shape[0]
        _check(host_lib().onn_trainer_step_host(self._handle, host_ptr(dec_ids), host_ptr(enc_ids), host_ptr(targets),
                                                C.c_int64(batch), int(update), stats if want_statistics else None), "step_host")
        return tuple(stats) if want_statistics else None

    def step_host_i32(self, dec_ids, enc_ids, targets, update=True, want_statistics=True):
        """Same, fed with int32 ids in host memory (torch CPU tensors, pinned for full copy speed): the ids are copied
        on a copy stream into one of two sets of device buffers and converted on the device."""
        import torch
        stats = (C.c_float * 4)()
        for x in (dec_ids, enc_ids, targets):
            if x is not None and (x.dtype != torch.int32 or not x.is_contiguous() or x.is_cuda):
                raise ValueError("step_host_i32 takes contiguous int32 CPU tensors")
        batch = dec_ids.shape[0]
        _check(host_lib().onn_trainer_step_host_i32(self._handle, C.c_void_p(dec_ids.data_ptr()),
                                                    C.c_void_p(enc_ids.data_ptr() if enc_ids is not None else 0),
                                                    C.c_void_p(targets.data_ptr()), C.c_int64(batch), int(update),
                                                    stats if want_statistics else None), "step_host_i32")
        return tuple(stats) if want_statistics else None

    def forward(self, dec_ids, enc_ids, is_training=False):
        _check(host_lib().onn_trainer_forward(self._handle, capi.ptr(dec_ids), capi.ptr(enc_ids), int(is_training)), "forward")

    def greedy_decode(self, encoder_ids, start_id=2, end_id=3, cached=False):
        """encoder_ids: float32 numpy [micro_batch, S_in]; returns float32 numpy [micro_batch, S_dec].
        cached=True decodes one position per step with cached keys and values."""
        encoder_ids = np.ascontiguousarray(encoder_ids, dtype=np.float32)
        decoded = np.zeros((encoder_ids.shape[0], self.S_dec), dtype=np.float32)
        entry = host_lib().onn_trainer_greedy_decode_cached if cached else host_lib().onn_trainer_greedy_decode
        _check(entry(self._handle, _f32_ptr(encoder_ids), _f32_ptr(decoded), int(start_id), int(end_id)), "greedy_decode")
        return decoded

    def layer_output(self, i, count=None):
        _, _, _, size = self.layer_info(i)
        count = size if count is None else count
        a = np.empty(count, dtype=np.float32)
        _check(host_lib().onn_trainer_get_layer_output(self._handle, int(i), _f32_ptr(a), C.c_int64(count)), "get_layer_output")
        return a

    def stream(self):
        """torch view of the CUDA stream the trainer launches on (for torch.cuda.Event timing)."""
        import torch
        return torch.cuda.ExternalStream(host_lib().onn_trainer_stream(self._handle))

    def synchronize(self):
        _check(host_lib().onn_trainer_synchronize(self._handle), "synchronize")

    def exchange_segments(self):
        return int(host_lib().onn_trainer_exchange_segments(self._handle))

    def trace_phases(self, enabled=True):
        _check(host_lib().onn_trainer_trace_phases(self._handle, int(bool(enabled))), "trace_phases")

    def last_step_phases(self):
        """Milliseconds {start -> forward pass done, back-propagation, update} of the last traced step."""
        out = (C.c_float * 3)()
        _check(host_lib().onn_trainer_last_step_phases(self._handle, out), "last_step_phases")
        return [float(x) for x in out]

    def parameters_ready(self):
        """Makes the trainer's stream wait for the parameter all-gathers a data-parallel step left in flight."""
        _check(host_lib().onn_trainer_parameters_ready(self._handle), "parameters_ready")


class TextClassifier:
    """TextClassificationNetwork + CrossEntropyError2d + Adam on the current CUDA device: Embedding -> self-attention ->
    max pooling over the sequence -> Dense<2> ReLU layers -> Dense<2> Softmax."""

    def __init__(self, V, S, E, H, hidden, classes, batch):
        self.S, self.classes, self.batch = S, classes, batch
        self._handle = C.c_void_p()
        i64 = C.c_int64
        sizes = (i64 * max(len(hidden), 1))(*hidden)
        status = host_lib().onn_classifier_create(C.byref(self._handle), i64(V), i64(S), i64(E), i64(H), sizes, len(hidden), i64(classes), i64(batch))
        self._check(status, "onn_classifier_create")
        self.parameters_number = int(host_lib().onn_classifier_parameters_number(self._handle))
        self.layers_number = int(host_lib().onn_classifier_layers_number(self._handle))

    @staticmethod
    def _check(status, what):
        if status != 0:
            raise capi.OnnError(f"{what}: {host_lib().onn_classifier_last_error().decode()} ({status})")

    def close(self):
        if self._handle:
            host_lib().onn_classifier_destroy(self._handle)
            self._handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def layer_info(self, i):
        name, label = C.create_string_buffer(128), C.create_string_buffer(128)
        params = C.c_int64()
        self._check(host_lib().onn_classifier_layer_info(self._handle, int(i), name, label, 128, C.byref(params)), "layer_info")
        return name.value.decode(), label.value.decode(), params.value

    def set_parameters(self, host_array):
        a = np.ascontiguousarray(host_array, dtype=np.float32)
        assert a.size == self.parameters_number
        self._check(host_lib().onn_classifier_set_parameters(self._handle, _f32_ptr(a)), "set_parameters")

    def get_parameters(self):
        a = np.empty(self.parameters_number, dtype=np.float32)
        self._check(host_lib().onn_classifier_get_parameters(self._handle, _f32_ptr(a)), "get_parameters")
        return a

    def get_gradients(self):
        a = np.empty(self.parameters_number, dtype=np.float32)
        self._check(host_lib().onn_classifier_get_gradients(self._handle, _f32_ptr(a)), "get_gradients")
        return a

    def set_learning_rate(self, lr):
        self._check(host_lib().onn_classifier_set_learning_rate(self._handle, C.c_float(lr)), "set_learning_rate")

    def set_dp(self, comm_handle, world):
        """Data-parallel training: every rank steps its own `batch` samples; gradients and the error are averaged
        over the ranks before the update (get_gradients then returns the SUM over ranks)."""
        self._check(host_lib().onn_classifier_set_dp(self._handle, comm_handle, int(world)), "set_dp")

    def layer_output(self, i):
        """Output of layer i after the last forward pass, as a flat float32 array."""
        a = np.empty(int(host_lib().onn_classifier_layer_output_size(self._handle, int(i))), dtype=np.float32)
        self._check(host_lib().onn_classifier_get_layer_output(self._handle, int(i), _f32_ptr(a), C.c_int64(a.size)), "get_layer_output")
        return a

    def forward(self, ids):
        """ids: torch CUDA float tensor [batch, S].  Returns the class probabilities [batch, classes] (numpy)."""
        assert tuple(ids.shape) == (self.batch, self.S)
        out = np.empty((self.batch, self.classes), dtype=np.float32)
        self._check(host_lib().onn_classifier_forward(self._handle, capi.ptr(ids), _f32_ptr(out)), "forward")
        return out

    def step_device(self, ids, targets, update=True):
        """ids [batch, S], targets [batch, classes] one-hot: torch CUDA float tensors.  Returns (error, gradient norm)."""
        assert tuple(ids.shape) == (self.batch, self.S) and tuple(targets.shape) == (self.batch, self.classes)
        stats = (C.c_float * 2)()
        self._check(host_lib().onn_classifier_step_device(self._handle, capi.ptr(ids), capi.ptr(targets), int(update), stats), "step_device")
        return tuple(stats)


def shard_batch(arrays, rank, world):
    """The data-parallel rule of the trainer for a batch every rank can see: rank r of `world` takes the r-th of
    `world` equal contiguous slices of each array's first dimension (the global batch must divide evenly, so that
    every rank runs the same number of micro-batches and joins the same collectives)."""
    shards = []
    for a in arrays:
        if a is None:
            shards.append(None)
            continue
        if a.shape[0] % world != 0:
            raise ValueError(f"batch of {a.shape[0]} samples does not split evenly over {world} ranks")
        share = a.shape[0] // world
        shards.append(a[rank * share:(rank + 1) * share])
    return shards


def shard_layout(parameters, world, bucket_floats=16 << 20):
    """The partition the sharded data-parallel update works on (the trainer's C++ side computes the same): the arena
    is rounded up to a multiple of 4 * world floats (`total`) and cut on a fixed grid into buckets of `bucket` floats
    (itself a multiple of 4 * world); rank r owns the r-th of `world` equal parts of every bucket, so every part
    starts on a 16-byte boundary.  Returns (total, bucket, [(low, part)] per bucket): rank r's share of a bucket is
    arena[low + r * part : low + (r + 1) * part], kept compactly at own[low // world : low // world + part]."""
    unit = 4 * world
    total = (parameters + unit - 1) // unit * unit
    bucket = max(unit, bucket_floats // unit * unit)
    parts = []
    low = 0
    while low < total:
        size = min(bucket, total - low)
        parts.append((low, size // world))
        low += size
    return total, bucket, parts


class DpRendezvousError(RuntimeError):
    """A data-parallel job that must not start: a rank is missing or the replicas differ."""


def dp_check_replicas(signature, timeout_s=60.0):
    """Failure detection on the host, before any NCCL call or kernel launch (the reference has no multi-GPU path, so
    there is no counterpart): every rank of the initialised torch.distributed group publishes `signature` (anything
    picklable that must be equal on all replicas: parameter count, micro-batch, network shape) in the group's store
    and waits at most `timeout_s` seconds for the others.  Raises DpRendezvousError naming the ranks that never
    arrived, or the first rank whose signature differs from rank 0's.  Every rank sees the same data, so every rank
    that arrived raises the same error and none of them goes on to wait in a collective for the others."""
    import datetime
    import pickle
    import torch.distributed as dist
    world, rank = dist.get_world_size(), dist.get_rank()
    store = dist.distributed_c10d._get_default_store()
    generation = dp_check_replicas.generation = getattr(dp_check_replicas, "generation", 0) + 1
    keys = [f"onn_b200/replica/{generation}/{r}" for r in range(world)]
    store.set(keys[rank], pickle.dumps(signature))
    try:
        store.wait(keys, datetime.timedelta(seconds=float(timeout_s)))
    except Exception as error:                                   # the store raises its own timeout type
        missing = [r for r in range(world) if not store.check([keys[r]])]
        raise DpRendezvousError(f"rank {rank}: ranks {missing} did not join within {timeout_s} s") from error
    published = [pickle.loads(store.get(key)) for key in keys]
    for r, other in enumerate(published):
        if other != published[0]:
            raise DpRendezvousError(f"rank {rank}: replica {r} differs from replica 0: {other!r} != {published[0]!r}")
    return published[0]


def dp_init_from_torch(signature=None, timeout_s=60.0, max_ctas=None):
    """Creates the NCCL communicator of libonn_b200 for the ranks of an initialised
    torch.distributed process group (the 128-byte unique id travels through it).  The ranks first check
    on the host that all of them are present and hold the same replica (dp_check_replicas on `signature`;
    without one, on the number of ranks alone), so a missing rank or a mismatched parameter arena ends the
    job with an error instead of a wait without limit inside ncclCommInitRank or a corrupted all-reduce.
    max_ctas caps the SMs NCCL's kernels may use (default: ONN_B200_DP_MAX_CTAS, else NCCL's own choice)."""
    import torch
    import torch.distributed as dist
    world, rank = dist.get_world_size(), dist.get_rank()
    dp_check_replicas(signature if signature is not None else {"world": world}, timeout_s)
    if max_ctas is None:
        max_ctas = int(os.environ.get("ONN_B200_DP_MAX_CTAS", "0") or 0)
    uid = (C.c_char * 128)()
    if rank == 0:
        capi.check(capi.lib().onn_dp_unique_id(uid), "onn_dp_unique_id")
    payload = [bytes(uid.raw)]
    dist.broadcast_object_list(payload, src=0)
    uid_buffer = (C.c_char * 128).from_buffer_copy(payload[0])
    comm = C.c_void_p()
    capi.check(capi.lib().onn_dp_init_config(C.byref(comm), uid_buffer, int(world), int(rank), int(max_ctas)), "onn_dp_init_config")
    return comm
