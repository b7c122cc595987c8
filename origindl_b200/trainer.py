"""Host-side driver of the device-resident MLP training state (odl_mlp_* in include/odl_b200.h).

Mirrors the reference's training loop (tests/example/mnist/mlp_mnist.cpp:176-437):

    model = nn::MLP(sizes); optimizer = Adam(model, lr); optimizer.register_hook(WeightDecay(rate).hook())
    y = model(x); loss = softmax_cross_entropy(y, t); optimizer.zero_grad(); loss.backward(); optimizer.step()

Data parallelism (one process per GPU): every rank holds full parameter / optimizer replicas and its own slice of
the batch.  After layer l's backward the rank's gradient bucket [dW_l, db_l] -- one contiguous range of the flat
gradient buffer -- is summed across ranks with NCCL on a side stream while layers l-1 ... 0 keep computing; the
optimizer then scales by 1/world_size inside its fused update.  By default the whole data-parallel step, collectives
included, is ONE call into the library (odl_mlp_train_step_dp: the library owns the communicator, the communication
stream and the events, so a C++ host runs the very same step); the process group is then only the channel that hands
NCCL's rendezvous token to the other ranks.  `native_dp=False` keeps the older driver that issues the same all-reduces
through torch.distributed from Python (same bits).  All arithmetic is in libodl_b200.so.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import capi, dp


class MLPTrainer:
    def __init__(self, sizes, batch, optimizer="adam", lr=1e-3, momentum=0.0, hook_weight_decay=0.0,
                 precision=capi.PRECISION_3XTF32, device=0, process_group=None, overlap=True, native_dp=True,
                 dw0_panels=0):
        capi.init(device)
        self.sizes = [int(s) for s in sizes]
        self.batch = int(batch)
        self.n_layers = len(self.sizes) - 1
        self.optimizer, self.lr = optimizer, float(lr)
        arr = (ctypes.c_int32 * len(self.sizes))(*self.sizes)
        h = ctypes.c_void_p()
        opt = {"sgd": 0, "adam": 1}[optimizer]
        capi.call("odl_mlp_create", arr, len(self.sizes), self.batch, opt, lr, momentum, hook_weight_decay, precision,
                  ctypes.byref(h))
        self._h = h
        self.pg = process_group
        self.world = 1
        self.overlap = overlap
        self._buckets = None
        self._comm = None
        if process_group is not None:
            import torch.distributed as dist

            self.world = dist.get_world_size(process_group)
            if native_dp and overlap:
                # the library's own communicator: rank 0 makes NCCL's rendezvous token, the process group carries it
                token = ctypes.create_string_buffer(128)
                if dist.get_rank(process_group) == 0:
                    capi.call("odl_comm_unique_id", token)
                box = [token.raw]
                dist.broadcast_object_list(box, src=dist.get_global_rank(process_group, 0), group=process_group)
                comm = ctypes.c_void_p()
                capi.call("odl_comm_create", box[0], dist.get_rank(process_group), self.world, ctypes.byref(comm))
                self._comm = comm
                capi.call("odl_mlp_dp_attach", self._h, self._comm, int(dw0_panels))
            else:
                self._comm_stream = torch.cuda.Stream()
                self._buckets = [self._bucket_tensor(l) for l in range(self.n_layers)]
        self._loss_view = self._view(capi.lib().odl_mlp_loss_ptr(self._h), 1)

    # -- raw device memory of the library wrapped as torch tensors (no copy) so that NCCL can reduce it in place
    @staticmethod
    def _view(ptr: int, count: int) -> torch.Tensor:
        class _Blob:
            pass

        b = _Blob()
        b.__cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (ptr, False), "version": 3,
                                      "strides": None}
        return torch.as_tensor(b, device="cuda")

    def _bucket_tensor(self, layer: int) -> torch.Tensor:
        p, n = ctypes.c_void_p(), ctypes.c_int64()
        capi.call("odl_mlp_grad_bucket", self._h, layer, ctypes.byref(p), ctypes.byref(n))
        return self._view(p.value, n.value)

    @property
    def param_count(self) -> int:
        return int(capi.lib().odl_mlp_param_count(self._h))

    def set_params(self, packed: np.ndarray) -> None:
        packed = np.ascontiguousarray(packed, np.float32)
        assert packed.size == self.param_count
        capi.call("odl_mlp_set_params", self._h, packed.ctypes.data, capi.stream_handle())

    def get_params(self) -> np.ndarray:
        out = np.empty(self.param_count, np.float32)
        capi.call("odl_mlp_get_packed", self._h, 0, out.ctypes.data, capi.stream_handle())
        return out

    def get_grads(self) -> np.ndarray:
        out = np.empty(self.param_count, np.float32)
        capi.call("odl_mlp_get_packed", self._h, 1, out.ctypes.data, capi.stream_handle())
        return out

    # -- state dict / checkpoint in the reference's formats (Module::state_dict, src/nn/module.cpp:118-128; origin::save
    #    of a Checkpoint, src/io/checkpoint.cpp:15-75).  Names and shapes are those of nn::MLP: layer_i.weight {in,out},
    #    layer_i.bias {1,out} (src/nn/models/mlp.cpp:21-34, src/nn/layers/linear.cpp:25-62).
    def _named_shapes(self):
        for i in range(self.n_layers):
            yield f"layer_{i}.weight", (self.sizes[i], self.sizes[i + 1])
            yield f"layer_{i}.bias", (1, self.sizes[i + 1])

    def _unpack(self, packed: np.ndarray, prefix: str = "") -> dict:
        out, o = {}, 0
        for name, shape in self._named_shapes():
            n = shape[0] * shape[1]
            out[prefix + name] = packed[o:o + n].reshape(shape)
            o += n
        return out

    def _pack(self, tensors: dict, prefix: str = "", strict: bool = True) -> np.ndarray:
        packed = np.empty(self.param_count, np.float32) if strict else self.get_params()
        o = 0
        for name, shape in self._named_shapes():
            n = shape[0] * shape[1]
            t = tensors.get(prefix + name)
            if t is None:
                if strict:
                    raise RuntimeError(f"Missing parameter '{prefix + name}' in state_dict (strict mode)")
            else:
                if tuple(t.shape) != shape:
                    raise RuntimeError(f"Shape mismatch for parameter '{prefix + name}': expected {shape}, got {tuple(t.shape)}")
                packed[o:o + n] = np.asarray(t, np.float32).reshape(-1)
            o += n
        return packed

    def state_dict(self) -> dict:
        return self._unpack(self.get_params())

    def load_state_dict(self, state_dict: dict, strict: bool = True) -> None:
        """Module::load_state_dict (src/nn/module.cpp:130-168): shape mismatches always raise; missing and unexpected
        names raise in strict mode.  Installing parameters resets the optimizer state (load it afterwards)."""
        if strict:
            known = {n for n, _ in self._named_shapes()}
            for key in state_dict:
                if key not in known:
                    raise RuntimeError(f"Unexpected parameter '{key}' in state_dict (strict mode)")
        self.set_params(self._pack(state_dict, strict=strict))

    def optimizer_state_dict(self) -> dict:
        """m_<param>, v_<param> (Adam only) and step_<param>: the keys of Adam::state_dict (src/optim/adam.cpp:116-193)."""
        buf = np.empty(self.param_count, np.float32)
        capi.call("odl_mlp_get_packed", self._h, 2, buf.ctypes.data, capi.stream_handle())
        out = self._unpack(buf.copy(), "m_")
        if self.optimizer == "adam":
            capi.call("odl_mlp_get_packed", self._h, 3, buf.ctypes.data, capi.stream_handle())
            out.update(self._unpack(buf.copy(), "v_"))
        step = int(capi.lib().odl_mlp_step_count(self._h))
        for name, _ in self._named_shapes():
            out["step_" + name] = np.array([step], np.int32)
        return out

    def load_optimizer_state_dict(self, state: dict) -> None:
        m = self._pack(state, "m_")
        v = self._pack(state, "v_") if self.optimizer == "adam" else None
        steps = {int(np.asarray(state["step_" + n]).reshape(-1)[0]) for n, _ in self._named_shapes()}
        if len(steps) != 1:
            raise RuntimeError(f"optimizer state holds different step counts per parameter: {sorted(steps)}")
        capi.call("odl_mlp_set_optimizer_state", self._h, m.ctypes.data, None if v is None else v.ctypes.data,
                  steps.pop(), capi.stream_handle())

    def save_checkpoint(self, filepath: str, epoch: int = -1, step: int = -1, loss: float = 0.0) -> str:
        from . import odl_io

        cfg = {"lr": self.lr}
        if self.optimizer == "adam":
            cfg.update(beta1=0.9, beta2=0.999, eps=1e-8)
        ck = odl_io.Checkpoint(self.state_dict(), self.optimizer_state_dict(), epoch, step, loss,
                               {"adam": "Adam", "sgd": "SGD"}[self.optimizer], cfg)
        return odl_io.save_checkpoint(ck, filepath, (odl_io.DEVICE_CUDA, torch.cuda.current_device()))

    def load_checkpoint(self, filepath: str):
        """Restore parameters and, when the checkpoint holds it, the optimizer state; returns the Checkpoint."""
        from . import odl_io

        ck = odl_io.load_checkpoint(filepath)
        self.load_state_dict(ck.model_state_dict)
        if ck.optimizer_state_dict:
            self.load_optimizer_state_dict(ck.optimizer_state_dict)
        return ck

    def logits(self) -> torch.Tensor:
        return self._view(capi.lib().odl_mlp_logits_ptr(self._h), self.batch * self.sizes[-1]).view(self.batch, -1)

    def loss_tensor(self) -> torch.Tensor:
        """0-dim view of the device loss of the last forward (no synchronisation)."""
        return self._loss_view[0]

    def train_step(self, x: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        """One optimisation step on x[batch, sizes[0]] / labels[batch]; returns the device loss (a view)."""
        assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and tuple(x.shape) == (self.batch, self.sizes[0])
        assert labels.is_cuda and labels.is_contiguous() and labels.dtype in (torch.int32, torch.int64)
        s = capi.stream_handle()
        is64 = int(labels.dtype == torch.int64)
        if self.pg is None:
            capi.call("odl_mlp_train_step", self._h, x.data_ptr(), labels.data_ptr(), is64, s)
            return self._loss_view[0]
        if self._comm is not None:
            capi.call("odl_mlp_train_step_dp", self._h, x.data_ptr(), labels.data_ptr(), is64, s)
            return self._loss_view[0]
        import torch.distributed as dist

        compute = torch.cuda.current_stream()
        capi.call("odl_mlp_forward_loss", self._h, x.data_ptr(), labels.data_ptr(), is64, s)
        reduced = {}
        for layer in dp.reduce_order(self.n_layers):
            capi.call("odl_mlp_backward_layer", self._h, layer, s)
            if self.overlap:
                ev = torch.cuda.Event()
                ev.record(compute)
                self._comm_stream.wait_event(ev)
                with torch.cuda.stream(self._comm_stream):
                    dist.all_reduce(self._buckets[layer], op=dist.ReduceOp.SUM, group=self.pg)
                    reduced[layer] = torch.cuda.Event()
                    reduced[layer].record(self._comm_stream)
        if not self.overlap:
            for layer in range(self.n_layers - 1, -1, -1):
                dist.all_reduce(self._buckets[layer], op=dist.ReduceOp.SUM, group=self.pg)
            capi.call("odl_mlp_optimizer_step", self._h, 1.0 / self.world, s)
            return self._loss_view[0]
        # update each layer as soon as ITS bucket is reduced: the head-side layers' updates run while the last bucket
        # (layer 0, whose gradient is the last GEMM of backward) is still being reduced
        for i, layer in enumerate(dp.reduce_order(self.n_layers)):
            compute.wait_event(reduced[layer])
            capi.call("odl_mlp_optimizer_step_layer", self._h, layer, 1.0 / self.world, int(i == 0), s)
        return self._loss_view[0]

    def capture(self, x: torch.Tensor, labels: torch.Tensor):
        """Capture forward + loss + backward on the given STATIC input buffers into one CUDA graph and return a
        function that runs one optimisation step: graph replay, then the optimizer launch (kept outside the graph
        because Adam's bias corrections are host scalars that change every step).  The caller refills `x` / `labels`
        in place between steps.  Two eager warm-up steps run first so that the scratch arena has its final size
        before capture (allocation is not capturable).  Single-GPU only."""
        if self.pg is not None:
            raise NotImplementedError("graph capture of the data-parallel step is not implemented")
        assert x.is_cuda and x.is_contiguous() and tuple(x.shape) == (self.batch, self.sizes[0])
        is64 = int(labels.dtype == torch.int64)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            for _ in range(2):
                self.train_step(x, labels)
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                s = capi.stream_handle()
                capi.call("odl_mlp_forward_loss", self._h, x.data_ptr(), labels.data_ptr(), is64, s)
                for layer in dp.reduce_order(self.n_layers):
                    capi.call("odl_mlp_backward_layer", self._h, layer, s)
        torch.cuda.current_stream().wait_stream(side)
        generation = capi.lib().odl_scratch_generation()

        def step() -> torch.Tensor:
            # the graph holds addresses inside the library's scratch blocks; a later call that made them grow replaced them
            if capi.lib().odl_scratch_generation() != generation:
                raise capi.OdlError(capi.ERR_STALE_GRAPH, "the library's scratch memory was replaced after capture(); "
                                                          "capture the step again")
            graph.replay()
            capi.call("odl_mlp_optimizer_step", self._h, 1.0, capi.stream_handle())
            return self._loss_view[0]

        return step

    def capture_native(self, x: torch.Tensor, labels: torch.Tensor):
        """The same whole-step graph recorded by the library itself (odl_mlp_capture / odl_mlp_replay -- what a C++ host
        uses): returns a function that runs one optimisation step on the STATIC buffers `x` / `labels`.  Single-GPU only."""
        if self.pg is not None:
            raise NotImplementedError("graph capture of the data-parallel step is not implemented")
        assert x.is_cuda and x.is_contiguous() and tuple(x.shape) == (self.batch, self.sizes[0])
        is64 = int(labels.dtype == torch.int64)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        capi.call("odl_mlp_capture", self._h, x.data_ptr(), labels.data_ptr(), is64, side.cuda_stream)
        side.synchronize()

        def step() -> torch.Tensor:
            side.wait_stream(torch.cuda.current_stream())  # the caller refilled x / labels on its own stream
            capi.call("odl_mlp_replay", self._h, side.cuda_stream)
            torch.cuda.current_stream().wait_stream(side)
            return self._loss_view[0]

        return step

    def wait(self, timeout_ms: int = 60000) -> None:
        """Host watchdog over the last data-parallel step: returns once its last all-reduce has completed; raises
        OdlError (ERR_COMM / ERR_COMM_TIMEOUT) and aborts the communicator when NCCL reports an asynchronous error or
        the collective does not complete in time (a peer that never joined).  Native data-parallel mode only."""
        if self._comm is None:
            raise RuntimeError("wait() needs the library's own communicator (process_group given, native_dp=True)")
        capi.call("odl_mlp_dp_wait", self._h, int(timeout_ms))

    def comm_status(self) -> None:
        """Raise OdlError(ERR_COMM) if NCCL has noticed an asynchronous error on the library's communicator."""
        if self._comm is not None:
            capi.call("odl_comm_status", self._comm)

    def close(self) -> None:
        if self._h is not None:
            capi.call("odl_mlp_destroy", self._h)
            self._h = None
        if self._comm is not None:
            capi.call("odl_comm_destroy", self._comm)
            self._comm = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
