"""A decode step with host-resident activations as ONE CUDA graph: pinned host inputs -> device copy -> the step's quantized linears -> copy of the results
into pinned host buffers. The reference reaches the same effect with MLX's lazy graph (one `mx.eval` per step; kyojin_mlx/foreign_linear.py:67 notes the tens of
microseconds of Python dispatch per call that this removes); here the launch-bound inner loop is captured once and replayed.

    step = HostGraph(lambda x: [lin_q(x), lin_k(x)], [(4, 5120)])          # input shapes (float16); captures on the current device
    step.inputs[0].copy_(new_activations)                                  # pinned host views: the caller writes the step's activations in place
    outs = step()                                                          # replay + wait; list of pinned host tensors, valid until the next call

A step may be given as several stages, `HostGraph.staged([(fn_a, shapes_a), (fn_b, shapes_b), ...])`: the stages run in order on the compute stream while the
inputs of later stages are uploaded and the results of earlier stages are downloaded on two copy streams inside the same graph, so only the first upload and the
last download are exposed. `inputs` / `outputs` are then lists over all stages, in order.
Every stage moves its activations with one host-to-device copy and its results with one device-to-host copy (one pinned buffer each)."""
from __future__ import annotations

import torch


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


def _nbytes(shape, dtype) -> int:
    return int(torch.Size(shape).numel()) * torch.empty((), dtype=dtype).element_size()


def _view(buf, off, shape, dtype):
    return buf[off:off + _nbytes(shape, dtype)].view(dtype).reshape(shape)


class _Stage:
    def __init__(self, fn, inputs, device, dtype):
        given = [i for i in inputs if isinstance(i, torch.Tensor)]
        if given and any(not h.is_pinned() for h in given):
            raise ValueError("host inputs must be pinned (page-locked) tensors")
        self.fn = fn
        shapes = [tuple(i.shape) if isinstance(i, torch.Tensor) else tuple(i) for i in inputs]
        dts = [i.dtype if isinstance(i, torch.Tensor) else dtype for i in inputs]
        offs, total = [], 0
        for sh, dt in zip(shapes, dts):
            offs.append(total)
            total += _align(_nbytes(sh, dt))
        self.hin = torch.empty(max(total, 256), dtype=torch.uint8).pin_memory()
        self.din = torch.empty(max(total, 256), dtype=torch.uint8, device=device)
        self.inputs = [_view(self.hin, o, sh, dt) for o, sh, dt in zip(offs, shapes, dts)]
        self.dviews = [_view(self.din, o, sh, dt) for o, sh, dt in zip(offs, shapes, dts)]
        for v, i in zip(self.inputs, inputs):
            if isinstance(i, torch.Tensor):
                v.copy_(i)
        self.hout = self.dout = self.oviews = self.outputs = None
        self.device = device

    def compute(self):
        """Runs the stage on the current stream and gathers its results into one device buffer."""
        from . import ops
        outs = self.fn(*self.dviews)
        outs = [outs] if isinstance(outs, torch.Tensor) else list(outs)
        if self.hout is None:
            oo, tot = [], 0
            for o in outs:
                oo.append(tot)
                tot += _align(o.numel() * o.element_size())
            self.dout = torch.empty(max(tot, 256), dtype=torch.uint8, device=self.device)
            self.hout = torch.empty(max(tot, 256), dtype=torch.uint8).pin_memory()
            self.oviews = [_view(self.dout, p, tuple(o.shape), o.dtype) for p, o in zip(oo, outs)]
            self.outputs = [_view(self.hout, p, tuple(o.shape), o.dtype) for p, o in zip(oo, outs)]
        pairs = list(zip(outs, self.oviews))
        fast = [(o, d) for o, d in pairs if o.is_contiguous() and (o.numel() * o.element_size()) % 16 == 0 and o.data_ptr() % 16 == 0]
        ops.gather_flat([o for o, _ in fast], [d for _, d in fast])          # one launch per 128 results
        for o, d in pairs:
            if not any(o is f for f, _ in fast):
                d.copy_(o)


class HostGraph:
    def __init__(self, fn, inputs, device=None, dtype=torch.float16, warmup: int = 2):
        """fn(*device_inputs) -> tensor or list of tensors, built from this package's modules / operators (no host synchronisation inside).
        inputs: shapes of the step's input tensors (of `dtype`), or pinned host tensors whose shapes and contents are taken over."""
        self._build([(fn, inputs)], device, dtype, warmup)

    @classmethod
    def staged(cls, stages, device=None, dtype=torch.float16, warmup: int = 2) -> "HostGraph":
        """stages: list of (fn, inputs); see the module text."""
        self = cls.__new__(cls)
        self._build(list(stages), device, dtype, warmup)
        return self

    def _build(self, stages, device, dtype, warmup):
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.stages = [_Stage(fn, inputs, self.device, dtype) for fn, inputs in stages]
        self.inputs = [v for st in self.stages for v in st.inputs]
        up, down = torch.cuda.Stream(device=self.device), torch.cuda.Stream(device=self.device)

        def body():
            cur = torch.cuda.current_stream(self.device)
            up.wait_stream(cur)
            down.wait_stream(cur)
            ready = []
            with torch.cuda.stream(up):                                      # uploads run ahead of the stages that need them
                for st in self.stages:
                    st.din.copy_(st.hin, non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(up)
                    ready.append(ev)
            for st, ev in zip(self.stages, ready):
                cur.wait_event(ev)
                st.compute()
                done = torch.cuda.Event()
                done.record(cur)
                with torch.cuda.stream(down):                                # the download of this stage overlaps the next stage
                    down.wait_event(done)
                    st.hout.copy_(st.dout, non_blocking=True)
            cur.wait_stream(up)
            cur.wait_stream(down)

        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):                                 # plans, workspaces and one-time attributes are set up outside the capture
                body()
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        # the capture runs on the warm-up stream: per-stream scratch (ops.workspace) set up by the warm-up is found again, so nothing is allocated inside the graph
        from . import ops
        self._side = side
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=side):
            body()
        self._scratch = ops._ws.get((self.device.index, side.cuda_stream))  # the graph holds this buffer's address: it lives as long as the graph
        self.outputs = [v for st in self.stages for v in st.outputs]
        self.h2d_bytes = sum(int(st.hin.numel()) for st in self.stages)
        self.d2h_bytes = sum(int(st.hout.numel()) for st in self.stages)

    def __del__(self):
        try:
            from . import ops
            ops.release_workspaces(self._side.cuda_stream)                  # the scratch cached for this graph's capture stream goes with the graph
        except Exception:
            pass

    def launch(self):
        """Replays the step without waiting (results are valid after a synchronisation of the current stream)."""
        self.graph.replay()
        return self.outputs

    def __call__(self):
        self.graph.replay()
        torch.cuda.current_stream(self.device).synchronize()
        return self.outputs
