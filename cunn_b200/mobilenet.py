"""Host side of the MobileNetV1 replica step and of the batch-sharded data-parallel step.

`MobileNetV1` owns the flat parameter / gradient / running-statistic buffers of one replica (torch
tensors provide the device memory) and calls `cunn_b200_mobilenet_step` in libTHCUNN.so.
`DataParallelStep` mirrors what nn.DataParallelTable does around such a replica
(DataParallelTable.lua): shard the batch with the reference's slice rule, run the replica, sum the
gradients over replicas, apply the same SGD update everywhere.  With one process per GPU the sum is an
NCCL all-reduce of the flat gradient buffer (torch.distributed is the plumbing).
"""
import ctypes

import numpy as np
import torch

from ._lib import lib, check, c_int, c_void_p, c_size_t, c_float, c_double

c_longlong = ctypes.c_longlong


class Config(ctypes.Structure):
    _fields_ = [("image_hw", c_int), ("width_div", c_int), ("num_classes", c_int)]


_P = ctypes.POINTER(Config)
lib.cunn_b200_mobilenet_param_count.restype = c_longlong
lib.cunn_b200_mobilenet_param_count.argtypes = [_P]
lib.cunn_b200_mobilenet_bn_stat_count.restype = c_longlong
lib.cunn_b200_mobilenet_bn_stat_count.argtypes = [_P]
lib.cunn_b200_mobilenet_num_layers.restype = c_int
lib.cunn_b200_mobilenet_num_layers.argtypes = [_P]
lib.cunn_b200_mobilenet_layer_info.restype = c_int
lib.cunn_b200_mobilenet_layer_info.argtypes = [_P, c_int, ctypes.POINTER(c_longlong)]
lib.cunn_b200_mobilenet_arena_bytes.restype = c_size_t
lib.cunn_b200_mobilenet_arena_bytes.argtypes = [_P, c_int]
lib.cunn_b200_mobilenet_step.restype = c_int
lib.cunn_b200_mobilenet_step.argtypes = [_P, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_size_t, c_void_p, c_double, c_double, c_void_p]

KIND_STEM, KIND_DW, KIND_PW, KIND_FC = 0, 1, 2, 3
_FIELDS = ("kind", "cin", "cout", "stride", "hin", "hout", "w_off", "b_off", "g_off", "beta_off", "bn_off", "wcount")


def slice_range(n, splits, idx):
    """Rows [start, start + count) of an n-row batch that replica idx (0-based) of `splits` receives: the
    first n mod splits replicas get one extra row (DataParallelTable.lua:469-479)."""
    per, extra = divmod(n, splits)
    if idx < extra:
        return idx * (per + 1), per + 1
    return extra * (per + 1) + (idx - extra) * per, per


def layout(cfg):
    """List of dicts describing every convolution (+ its BN) and, last, the classifier."""
    n = lib.cunn_b200_mobilenet_num_layers(ctypes.byref(cfg))
    if n < 0:
        raise ValueError("bad MobileNet configuration")
    out = []
    buf = (c_longlong * 12)()
    for i in range(n + 1):
        check(lib.cunn_b200_mobilenet_layer_info(ctypes.byref(cfg), i, buf))
        out.append(dict(zip(_FIELDS, [int(v) for v in buf])))
    return out


def init_params(cfg, seed=1234):
    """Seeded random initialisation on the host: convolution and classifier weights kaiming-uniform
    (bound 1/sqrt(fan_in)), biases uniform in the same bound, BN gamma ~ U(0,1), beta = 0."""
    rng = np.random.default_rng(seed)
    n = lib.cunn_b200_mobilenet_param_count(ctypes.byref(cfg))
    p = np.zeros(n, np.float32)
    for L in layout(cfg):
        if L["kind"] == KIND_DW:
            fan_in = 9
        elif L["kind"] == KIND_STEM:
            fan_in = L["cin"] * 9
        else:
            fan_in = L["cin"]
        bound = 1.0 / np.sqrt(fan_in)
        p[L["w_off"]:L["w_off"] + L["wcount"]] = rng.uniform(-bound, bound, L["wcount"])
        p[L["b_off"]:L["b_off"] + L["cout"]] = rng.uniform(-bound, bound, L["cout"])
        if L["kind"] != KIND_FC:
            p[L["g_off"]:L["g_off"] + L["cout"]] = rng.uniform(0, 1, L["cout"])
    return p


class MobileNetV1:
    """One replica: flat params / grads / BN running statistics on `device`."""

    def __init__(self, cfg, device, params_host, max_batch):
        self.cfg = cfg
        self.device = device
        self.nparams = lib.cunn_b200_mobilenet_param_count(ctypes.byref(cfg))
        self.params = torch.from_numpy(np.ascontiguousarray(params_host, dtype=np.float32)).to(device)
        self.grads = torch.zeros(self.nparams, device=device)
        nbn = lib.cunn_b200_mobilenet_bn_stat_count(ctypes.byref(cfg))
        self.bn_running = torch.zeros(nbn, device=device)
        for L in layout(cfg)[:-1]:                       # running_var starts at 1
            self.bn_running[L["bn_off"] + L["cout"]:L["bn_off"] + 2 * L["cout"]] = 1.0
        self.max_batch = max_batch
        nbytes = lib.cunn_b200_mobilenet_arena_bytes(ctypes.byref(cfg), max_batch)
        self.arena = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self.loss = torch.zeros(1, device=device)

    def zero_grad(self):
        self.grads.zero_()

    def step(self, images, labels, global_batch, momentum=0.1, eps=1e-5):
        """forward + loss + backward on the local rows; gradients of (1/global_batch) * sum NLL are
        accumulated into self.grads; returns the device scalar holding that scaled loss sum."""
        b = images.shape[0]
        if b > self.max_batch:
            raise ValueError("batch larger than the arena was sized for")
        check(lib.cunn_b200_mobilenet_step(ctypes.byref(self.cfg), images.data_ptr(), labels.data_ptr(), b,
                                           1.0 / global_batch, self.params.data_ptr(), self.grads.data_ptr(),
                                           self.bn_running.data_ptr(), self.arena.data_ptr(), self.arena.numel(),
                                           self.loss.data_ptr(), momentum, eps,
                                           torch.cuda.current_stream().cuda_stream))
        return self.loss

    def sgd(self, lr):
        check(lib.cunn_b200_sgd_update(self.params.data_ptr(), self.grads.data_ptr(), self.nparams, lr,
                                       torch.cuda.current_stream().cuda_stream))


class DataParallelStep:
    """Batch-sharded training step over the ranks of a torch.distributed process group (one process per
    GPU), with DataParallelTable's semantics: rank r takes slice_range(global_batch, world, r) of the batch,
    parameter gradients are SUMMED over replicas, BN statistics stay per shard, every replica applies the
    same update so parameters stay identical without a broadcast.  With dist=None it is a single replica."""

    def __init__(self, replica, dist=None, use_graph=False, native=True):
        """use_graph: replay zero_grad + forward + loss + backward from a CUDA graph (one per distinct pair of
        input buffers, batch and global batch; captured on the second use of the pair).  The ~300 launches of
        a step then cost one graph launch, which matters at small per-GPU batches.  The gradient all-reduce and
        the update stay outside the graph.
        native: with several ranks, the exchange and the update run in the library's DataParallelTable
        (cunn_b200_dpt_*: ncclAllReduce on a communication stream, visible += sum, update on every replica);
        torch.distributed then only carries the 128-byte NCCL id to the ranks.  native=False keeps
        torch.distributed.all_reduce."""
        self.replica = replica
        self.dist = dist
        self.world = dist.get_world_size() if dist is not None else 1
        self.rank = dist.get_rank() if dist is not None else 0
        self.use_graph = use_graph
        self._graphs = {}
        self._seen = set()
        self.table = None
        if native and self.world > 1 and replica.params.is_cuda:      # CPU stand-ins (gloo tests) keep the torch exchange
            from . import dpt
            dev = replica.params.device
            uid = torch.zeros(128, dtype=torch.uint8, device=dev)
            if self.rank == 0:
                uid.copy_(torch.frombuffer(bytearray(dpt.unique_id()), dtype=torch.uint8))
            dist.broadcast(uid, src=0)
            self.visible = torch.zeros_like(replica.grads)
            self.table = dpt.NativeDataParallelTable().add_rank(replica.nparams, dev.index, self.rank, self.world,
                                                               bytes(uid.cpu().numpy().tobytes()))
            self.table.set_buffers(0, replica.params.data_ptr(), replica.grads.data_ptr(), self.visible.data_ptr())

    def shard(self, global_batch):
        return slice_range(global_batch, self.world, self.rank)

    def train_step(self, images, labels, global_batch, lr):
        """images / labels: this rank's shard (already on its GPU)."""
        r = self.replica
        key = (images.data_ptr(), labels.data_ptr(), images.shape[0], global_batch)
        graph = self._graphs.get(key) if self.use_graph else None
        if graph is not None:
            graph.replay()
            loss = r.loss
        else:
            r.zero_grad()
            loss = r.step(images, labels, global_batch)
            if self.use_graph and images.shape[0] > 0 and len(self._graphs) < 8:
                if key in self._seen:
                    # second use of these buffers: the eager step above did this call's work, the capture only records
                    torch.cuda.current_stream().synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        r.zero_grad()
                        r.step(images, labels, global_batch)
                    self._graphs[key] = graph
                else:
                    self._seen.add(key)
        if self.table is not None:
            # visible = sum over the ranks of the local gradients (local is cleared), then the same update everywhere
            self.table.set_stream(0, torch.cuda.current_stream().cuda_stream)
            self.visible.zero_()
            self.table.reduce()
            self.table.updateParameters(lr)
            return loss
        if self.dist is not None and self.world > 1:
            self.dist.all_reduce(r.grads)
        r.sgd(lr)
        return loss
