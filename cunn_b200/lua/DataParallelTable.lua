--[[
 nn.DataParallelTable over the native table of libTHCUNN (include/cunn_b200_dpt.h).

 A thin LuaJIT-FFI shim with the constructor and method names of cunn's DataParallelTable.lua
 (nn.DataParallelTable(dimension, flattenParams, usenccl), :add, :threads, :forward, :backward,
 :zeroGradParameters, :updateParameters, :syncParameters, :getParameters, :training, :evaluate, :size, :get,
 torch.save / torch.load through __write / __read).  The container logic — shard rule, scatter, gather, gradient
 all-reduce in buckets on a communication stream, parameter broadcast, worker threads, watchdog, file format — is
 in C++ (cunn_b200/csrc/dpt.cu); this file only moves tensors' pointers across the FFI.

 NOT EXECUTED in this repository's tests: the image has no LuaJIT, cutorch or torch/nn.  It is written against the
 public cutorch / nn Lua API (torch.CudaTensor:data(), cutorch.setDevice, nn.Container) and is the file a Lua-Torch
 user would `require` in place of cunn's own DataParallelTable.lua.
]]--
local ffi = require 'ffi'
local C = ffi.load(package.searchpath('libTHCUNN', package.cpath))

ffi.cdef[[
typedef struct cunn_b200_dpt cunn_b200_dpt;
typedef void *cunn_stream_t;
const char *cunn_b200_last_error(void);
cunn_b200_dpt *cunn_b200_dpt_create(int dimension, int flatten_params, int use_nccl);
void cunn_b200_dpt_destroy(cunn_b200_dpt *t);
int cunn_b200_dpt_add(cunn_b200_dpt *t, const int *gpus, int ngpus, long long nparams);
int cunn_b200_dpt_threads(cunn_b200_dpt *t);
int cunn_b200_dpt_local_replicas(const cunn_b200_dpt *t);
int cunn_b200_dpt_replica_device(const cunn_b200_dpt *t, int replica);
int cunn_b200_dpt_set_buffers(cunn_b200_dpt *t, int replica, float *params, float *local_grads, float *visible_grads);
int cunn_b200_dpt_set_stream(cunn_b200_dpt *t, int replica, cunn_stream_t stream);
void cunn_b200_dpt_slice_range(long long n, int g, int i, long long *start, long long *count);
int cunn_b200_dpt_sync_parameters(cunn_b200_dpt *t);
int cunn_b200_dpt_zero_grad_parameters(cunn_b200_dpt *t);
int cunn_b200_dpt_update_parameters(cunn_b200_dpt *t, float lr);
int cunn_b200_dpt_reduce(cunn_b200_dpt *t);
int cunn_b200_dpt_watchdog(cunn_b200_dpt *t, double timeout_seconds);
int cunn_b200_dpt_write(cunn_b200_dpt *t, const char *path, const void *extra, long long extra_bytes);
int cunn_b200_dpt_read_params(cunn_b200_dpt *t, const char *path, void *extra);
]]

local function check(rc)
   if rc ~= 0 then error(ffi.string(C.cunn_b200_last_error()), 2) end
end

local DataParallelTable, parent = torch.class('nn.DataParallelTable', 'nn.Container')

function DataParallelTable:__init(dimension, flattenParams, usenccl)
   parent.__init(self)
   self.dimension = dimension or 1
   -- the library splits along the batch dimension only; its dimension argument is 0-based
   self.handle = ffi.gc(C.cunn_b200_dpt_create(self.dimension - 1, flattenParams and 1 or 0, usenccl and 1 or 0),
                        C.cunn_b200_dpt_destroy)
   if self.handle == nil then error(ffi.string(C.cunn_b200_last_error())) end
   self.gpuAssignments, self.replicas, self.visible = {}, {}, {}
   self.needsSync = true
end

-- :add(module, {gpu, ...}): one replica of `module` per listed GPU; their flat parameter / gradient vectors become the
-- table's buffers, a second gradient vector per replica receives the sum over replicas.
function DataParallelTable:add(module, gpus)
   local n = #gpus
   local ids = ffi.new('int[?]', n)
   for i = 1, n do ids[i - 1] = gpus[i] - 1; self.gpuAssignments[i] = gpus[i] end
   local nparams
   for i = 1, n do
      cutorch.withDevice(gpus[i], function()
         local replica = (i == 1) and module or module:clone()
         local p, g = replica:cuda():getParameters()          -- flattenParameters
         nparams = p:nElement()
         self.replicas[i] = {module = replica, params = p, grads = g}
         self.visible[i] = p.new(nparams):zero()
      end)
   end
   self.modules[1] = self.replicas[1].module
   check(C.cunn_b200_dpt_add(self.handle, ids, n, nparams))
   for i = 1, n do
      local r = self.replicas[i]
      check(C.cunn_b200_dpt_set_buffers(self.handle, i - 1, r.params:data(), r.grads:data(), self.visible[i]:data()))
   end
   return self
end

function DataParallelTable:threads() check(C.cunn_b200_dpt_threads(self.handle)); return self end
function DataParallelTable:size() return #self.replicas end
function DataParallelTable:get(i) return self.replicas[i].module end

local function slice(t, dim, n, g, i)
   local s, c = ffi.new('long long[1]'), ffi.new('long long[1]')
   C.cunn_b200_dpt_slice_range(n, g, i - 1, s, c)
   if c[0] == 0 then return nil end
   return t:narrow(dim, tonumber(s[0]) + 1, tonumber(c[0]))
end

function DataParallelTable:syncParameters()
   check(C.cunn_b200_dpt_sync_parameters(self.handle))
   self.needsSync = false
end

function DataParallelTable:updateOutput(input)
   if self.needsSync then self:syncParameters() end
   local g, n = #self.replicas, input:size(self.dimension)
   self.inputs, self.outputs = {}, {}
   for i = 1, g do
      cutorch.withDevice(self.gpuAssignments[i], function()
         local x = slice(input, self.dimension, n, g, i)
         if x then
            self.inputs[i] = x:cuda()
            self.outputs[i] = self.replicas[i].module:updateOutput(self.inputs[i])
         end
      end)
   end
   local parts = {}
   for i = 1, g do if self.outputs[i] then parts[#parts + 1] = self.outputs[i] end end
   self.output = torch.cat(parts, self.dimension)
   return self.output
end

function DataParallelTable:backward(input, gradOutput, scale)
   local g, n = #self.replicas, input:size(self.dimension)
   local parts = {}
   for i = 1, g do
      cutorch.withDevice(self.gpuAssignments[i], function()
         local gy = slice(gradOutput, self.dimension, n, g, i)
         if gy then parts[#parts + 1] = self.replicas[i].module:backward(self.inputs[i], gy:cuda(), scale) end
      end)
   end
   check(C.cunn_b200_dpt_reduce(self.handle))       -- visible += sum over replicas of the local gradients; local = 0
   self.gradInput = torch.cat(parts, self.dimension)
   return self.gradInput
end

function DataParallelTable:zeroGradParameters() check(C.cunn_b200_dpt_zero_grad_parameters(self.handle)) end
function DataParallelTable:updateParameters(lr) check(C.cunn_b200_dpt_update_parameters(self.handle, lr)) end
function DataParallelTable:getParameters() return self.replicas[1].params, self.visible[1] end

function DataParallelTable:training()
   for _, r in ipairs(self.replicas) do r.module:training() end
end

function DataParallelTable:evaluate()
   for _, r in ipairs(self.replicas) do r.module:evaluate() end
end

-- torch.save / torch.load: the table's own file (GPU assignment + replica 1's parameters) beside torch's stream
function DataParallelTable:__write(file)
   local path = os.tmpname()
   check(C.cunn_b200_dpt_write(self.handle, path, nil, 0))
   file:writeObject({gpuAssignments = self.gpuAssignments, module = self.replicas[1].module, table_file = path})
end
