"""nn.DataParallelTable for one process per GPU (reference: DataParallelTable.lua).

The reference keeps g replicas of a module inside one Lua process, scatters the input along `dimension`,
gathers the outputs on the first GPU, reduces the parameter gradients of replicas 2..g into replica 1 and
broadcasts replica 1's parameters before the next forward (`updateOutput :182-207`, `__backward :223-269`,
`syncParameters :283-294`).  Here every rank of a torch.distributed process group owns ONE replica on its own
GPU; the methods keep the reference's names and meaning, with these translations:

* scatter (`_distribute :527-578`): every rank is handed the full batch (or a tensor with the batch on dim 0)
  and keeps rows `sliceRange(n, g, rank)` (`:469-479`); a rank whose slice is empty runs no kernels but still
  takes part in the collectives (the reference uses fewer replicas when n < g, `:531`);
* gather (`_concat :583-623`): `forward` returns the LOCAL rows of the output; `gatherOutput()` concatenates the
  shards on every rank;
* reduce + broadcast: one all-reduce (sum) of the flat gradient buffer replaces reduce-to-replica-1
  (`:247-265`) and, because every rank then applies the same update, the broadcast of `syncParameters`
  is only needed after parameters were changed on one rank (load, manual edit): set `needsSync`.

Gradient accumulation over several `backward` calls between `zeroGradParameters` works as in the reference
(test_DataParallelTable.lua:531-576): the module accumulates into its LOCAL buffer `module.grads`; after each
backward the all-reduced sum is added to the VISIBLE buffer returned by `getParameters()` and the local buffer
is cleared, so no contribution is counted twice.

Module protocol (what `add` expects; `cunn_b200.mobilenet.MobileNetV1` adapters and the CPU stand-ins of the
tests provide it): attributes `params`, `grads` (flat fp32 tensors of equal length); `forward(input)`;
`backward(input, gradOutput, scale)` returning gradInput and accumulating `scale * dL/dparams` into `grads`;
optionally `training()` / `evaluate()`.
"""
import torch

from .mobilenet import slice_range


def sliceRange(nElem, idx, splits):
    """(start, size), start 0-based, of the rows that replica `idx` (1-based, like the reference) receives
    when `nElem` rows are dealt to `splits` replicas: DataParallelTable.lua:469-479."""
    return slice_range(nElem, splits, idx - 1)


class DataParallelTable:
    def __init__(self, dimension=1, flattenParams=True, usenccl=True, process_group=None, dist=None):
        if dimension != 1:
            raise ValueError("only the batch dimension (1) is sharded on this path")
        if not flattenParams:
            raise ValueError("parameters are always flat here (flattenParams = true)")
        self.dimension = dimension
        self.usenccl = usenccl
        self.dist = dist
        self.group = process_group
        self.world = dist.get_world_size(process_group) if dist is not None else 1
        self.rank = dist.get_rank(process_group) if dist is not None else 0
        self.module = None
        self.gradParameters = None      # visible gradient buffer: sum over replicas and over backward calls
        self.needsSync = True           # parameters may differ between ranks until the first sync
        self.output = None
        self.gradInput = None
        self.train = True

    # ---- construction ---------------------------------------------------------------------------------
    def add(self, module, gpus=None):
        """Registers this rank's replica.  `gpus` (the reference's GPU list) may be given for checking:
        its length must equal the number of ranks."""
        if self.module is not None:
            raise RuntimeError("one replica per process: add() was already called")
        if gpus is not None and len(gpus) != self.world:
            raise ValueError("%d GPUs listed but the process group has %d ranks" % (len(gpus), self.world))
        if module.params.numel() != module.grads.numel():
            raise ValueError("flat parameter and gradient buffers differ in length")
        self.module = module
        self.gradParameters = torch.zeros_like(module.grads)
        return self

    def size(self):
        return self.world

    def get(self, i):
        if i != self.rank + 1:
            raise IndexError("replica %d lives on rank %d" % (i, i - 1))
        return self.module

    def getParameters(self):
        return self.module.params, self.gradParameters

    def training(self):
        self.train = True
        if hasattr(self.module, "training"):
            self.module.training()

    def evaluate(self):
        self.train = False
        if hasattr(self.module, "evaluate"):
            self.module.evaluate()

    # ---- sharding -------------------------------------------------------------------------------------
    def shard(self, n):
        """(start, count) of this rank's rows of an n-row batch."""
        return sliceRange(n, self.rank + 1, self.world)

    def _local(self, t):
        s, c = self.shard(t.shape[0])
        return t.narrow(0, s, c)

    # ---- forward / backward ---------------------------------------------------------------------------
    def syncParameters(self):
        """Every replica takes replica 1's parameters (DataParallelTable.lua:283-294)."""
        if self.dist is not None and self.world > 1:
            self.dist.broadcast(self.module.params, src=0, group=self.group)
        self.needsSync = False

    def forward(self, input):
        if self.needsSync:
            self.syncParameters()
        x = self._local(input)
        self._input = x
        self.output = self.module.forward(x) if x.shape[0] > 0 else x.new_zeros((0,) + self._out_tail(input))
        return self.output

    updateOutput = forward

    def _out_tail(self, input):
        # shape of one output row, needed only by a rank without rows: ask the module if it knows
        if hasattr(self.module, "output_shape"):
            return tuple(self.module.output_shape(tuple(input.shape[1:])))
        return tuple(input.shape[1:])

    def gatherOutput(self, n):
        """The n-row output concatenated over the ranks (the reference's gather on GPU 1), on every rank."""
        out = self.output
        if self.dist is None or self.world == 1:
            return out
        counts = [sliceRange(n, r + 1, self.world)[1] for r in range(self.world)]
        width = max(counts)
        tail = tuple(out.shape[1:])
        padded = out.new_zeros((width,) + tail)
        padded[:out.shape[0]] = out
        parts = [torch.empty_like(padded) for _ in range(self.world)]
        self.dist.all_gather(parts, padded, group=self.group)
        return torch.cat([p[:c] for p, c in zip(parts, counts)], 0)

    def backward(self, input, gradOutput, scale=1.0):
        """updateGradInput + accGradParameters + gradient reduction; returns the local rows of gradInput."""
        x = self._local(input)
        gy = self._local(gradOutput)
        if x.shape[0] > 0:
            self.gradInput = self.module.backward(x, gy, scale)
        else:
            self.gradInput = x
        self._reduce()
        return self.gradInput

    def accGradParameters(self, input, gradOutput, scale=1.0):
        self.backward(input, gradOutput, scale)

    def _reduce(self):
        # visible += sum over replicas of the local buffers; local buffers start the next backward at zero
        local = self.module.grads
        if self.dist is not None and self.world > 1:
            self.dist.all_reduce(local, group=self.group)
        self.gradParameters += local
        local.zero_()

    def reduceLocal(self):
        """For modules that run forward, loss and backward in one fused call (the MobileNetV1 replica): folds the
        local gradient buffer into the visible one exactly like backward() does."""
        self._reduce()

    def zeroGradParameters(self):
        """Zeroes the gradients on ALL replicas (DataParallelTable.lua:300-313)."""
        self.module.grads.zero_()
        self.gradParameters.zero_()

    def updateParameters(self, learningRate):
        """p -= lr * g with the summed gradients, identically on every rank (DataParallelTable.lua:315-321)."""
        if hasattr(self.module, "sgd_with"):
            self.module.sgd_with(self.gradParameters, learningRate)
        else:
            self.module.params.add_(self.gradParameters, alpha=-learningRate)
