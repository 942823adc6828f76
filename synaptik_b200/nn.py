"""Python mirror of the reference's model-facing API for Linear/ReLU stacks.

``Model.compute`` and ``Model.train`` keep the names, argument meaning and observable results of
extensions/nn/.../module/Model.java:385,504 (compute: one forward run, result returned to the
host; train: one TRAINING_STEP run, objective returned, parameters updated in place) and of
``TrainingSession.runValues(..., RESET_AND_STEP)`` (modules/training/.../TrainingSession.java:568-642).
What differs is where state lives: parameters, gradients and optimizer moments stay in device
buffers between calls (the reference re-uploads every parameter and downloads every gradient per
step, TrainingSession.java:916-951, and lists device-resident parameters as future work,
docs/planning/native-performance-comparison.md:217-226).

Everything here goes through the C ABI (``native``); nothing computes on the host.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Sequence

import numpy as np

from . import native, program


@dataclass
class Sgd:
    learning_rate: float = 0.01
    momentum: float = 0.0
    dampening: float = 0.0
    weight_decay: float = 0.0
    nesterov: bool = False

    def native_kind(self):
        return native.SGD, [self.learning_rate, self.momentum, self.dampening, self.weight_decay, 1.0 if self.nesterov else 0.0]


@dataclass
class Adam:
    learning_rate: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    epsilon: float = 1e-8
    weight_decay: float = 0.0

    def native_kind(self):
        return native.ADAM, [self.learning_rate, self.beta1, self.beta2, self.epsilon, self.weight_decay]


@dataclass
class AdamW(Adam):
    def native_kind(self):
        return native.ADAMW, [self.learning_rate, self.beta1, self.beta2, self.epsilon, self.weight_decay]


def glorot_uniform(rng: np.random.Generator, out_features: int, in_features: int) -> np.ndarray:
    """U(-b, b), b = sqrt(6 / (fanIn + fanOut)) (ParameterInitializers.java:303-310); the reference
    draws (float)rng.nextDouble(lo, hi) (TensorRandoms.java:813)."""
    bound = math.sqrt(6.0 / (in_features + out_features))
    return rng.uniform(-bound, bound, size=(out_features, in_features)).astype(np.float32)


class Model:
    """A stack of ``Linear`` layers with ReLU between them (``ModelBuilder.linear().relu()...``).

    weights[l] is stored [out, in] like ``Linear`` (Linear.java:132-139); biases start at zero.
    """

    def __init__(self, dims: Sequence[int], context: native.Context | None = None, seed: int = 0,
                 comm: native.Comm | None = None, world_size: int = 1, bias: bool = True, activation: str = "relu",
                 dtype: str = "f32"):
        if activation not in ("relu", "tanh", "sigmoid", "silu", "gelu_tanh", "gelu"):
            raise ValueError("activation must be 'relu', 'tanh', 'sigmoid', 'silu', 'gelu_tanh' or 'gelu'")
        if dtype not in ("f32", "bf16", "f16"):
            raise ValueError("dtype must be 'f32', 'bf16' or 'f16'")
        # 16-bit storage (DataType.BFLOAT16 / FLOAT16): parameters, input and output are held as 16-bit values,
        # every node computes in FLOAT32 and narrows once; inference only (compute)
        self.dtype = dtype
        self.dims = list(dims)
        self.bias = bias
        self.activation = activation
        self.layers = len(self.dims) - 1
        self.context = context or native.Context(0)
        self.comm = comm
        self.world_size = world_size
        rng = np.random.default_rng(seed)
        self.param_buffers: List[native.Buffer] = []
        self.param_shapes: List[tuple] = []
        for l in range(self.layers):
            w = glorot_uniform(rng, self.dims[l + 1], self.dims[l])
            b = np.zeros(self.dims[l + 1], dtype=np.float32)
            for array in ((w, b) if bias else (w,)):
                self.param_buffers.append(self.context.upload(program.to_storage(self.dtype, array)))
                self.param_shapes.append(array.shape)
        self._inference = {}
        self._training = {}
        self._loss = None
        self._optimizer_config = None
        self._optimizer = None

    # ---- parameters -----------------------------------------------------------------------
    def parameters(self) -> List[np.ndarray]:
        """The parameters as FLOAT32 arrays (exactly the stored values, also for 16-bit storage)."""
        if self.dtype != "f32":
            return [program.from_storage(self.dtype, b.download(np.uint16, s)) for b, s in zip(self.param_buffers, self.param_shapes)]
        return [b.download(np.float32, s) for b, s in zip(self.param_buffers, self.param_shapes)]

    def load_parameters(self, arrays: Sequence[np.ndarray]) -> None:
        for buf, shape, array in zip(self.param_buffers, self.param_shapes, arrays):
            array = np.ascontiguousarray(array, dtype=np.float32)
            if array.shape != tuple(shape):
                raise ValueError(f"parameter shape {array.shape} != {shape}")
            buf.upload(program.to_storage(self.dtype, array))

    # ---- inference ------------------------------------------------------------------------
    def _inference_state(self, lead, arg_max: bool):
        key = (tuple(lead), arg_max)
        if key not in self._inference:
            graph = program.mlp_inference_graph(self.dims, tuple(lead), arg_max, bias=self.bias, activation=self.activation,
                                                dtype=program.STORAGE_DTYPES[self.dtype])
            exe = native.Executable(self.context, graph.image)
            batch = int(np.prod(lead))
            width = 4 if self.dtype == "f32" else 2
            x = self.context.buffer(batch * self.dims[0] * width)
            out = self.context.buffer(batch * self.dims[-1] * width)
            outs = [out] + ([self.context.buffer(batch * 8)] if arg_max else [])
            self._inference[key] = (exe, x, outs)
        return self._inference[key]

    def compute(self, x: np.ndarray, arg_max: bool = False):
        """Model.compute: uploads ``x`` [batch, in] (or [batch.., in]: every Linear applies to the last
        dimension), runs the forward graph, returns the output [batch.., out] (and the INT64 row arg-max
        when asked, for a [batch, in] input)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        if x.ndim < 2 or x.shape[-1] != self.dims[0]:
            raise ValueError(f"input shape {x.shape} does not end in {self.dims[0]} features")
        exe, xbuf, outs = self._inference_state(x.shape[:-1], arg_max)
        xbuf.upload(program.to_storage(self.dtype, x))
        exe.run([xbuf] + self.param_buffers, outs)
        if self.dtype != "f32":
            result = program.from_storage(self.dtype, outs[0].download(np.uint16, tuple(x.shape[:-1]) + (self.dims[-1],)))
        else:
            result = outs[0].download(np.float32, tuple(x.shape[:-1]) + (self.dims[-1],))
        if arg_max:
            return result, outs[1].download(np.int64, (x.shape[0],))
        return result

    # ---- training -------------------------------------------------------------------------
    def configure_training(self, loss: str, optimizer) -> None:
        """Model.configureTraining: ``loss`` is "ce" (index categorical cross entropy with logits,
        MEAN) or "mse" (MEAN); ``optimizer`` is Sgd, Adam or AdamW."""
        if loss not in ("ce", "mse"):
            raise ValueError("loss must be 'ce' or 'mse'")
        if self.dtype != "f32":
            raise ValueError("training needs FLOAT32 storage")
        self._loss = loss
        self._optimizer_config = optimizer
        kind, hyper = optimizer.native_kind()
        counts = [int(np.prod(s)) for s in self.param_shapes]
        self._optimizer = native.Optimizer(self.context, kind, hyper, self.param_buffers, counts)
        self._training = {}

    def training_state(self, batch: int):
        if self._loss is None:
            raise RuntimeError("configure_training first")
        if batch not in self._training:
            graph = program.mlp_training_graph(self.dims, batch, self._loss, bias=self.bias, activation=self.activation)
            exe = native.Executable(self.context, graph.image)
            x = self.context.buffer(batch * self.dims[0] * 4)
            t = self.context.buffer(batch * 4 if self._loss == "ce" else batch * self.dims[-1] * 4)
            # the seed scales the loss gradient; a data-parallel rank feeds 1/world so that the sum
            # of the ranks' gradients is the gradient of the global-batch mean
            seed = self.context.upload(np.array([1.0 / self.world_size], dtype=np.float32))
            loss = self.context.buffer(4)
            grads = [self.context.buffer(int(np.prod(s)) * 4) for s in self.param_shapes]
            if self.comm is not None:
                exe.attach_comm(self.comm, range(1, 1 + len(grads)))
            self._training[batch] = (exe, x, t, seed, loss, grads)
        return self._training[batch]

    def train(self, x: np.ndarray, target: np.ndarray, gradient_mode: int = native.Optimizer.RESET_AND_STEP) -> float:
        """Model.train / TrainingSession.runValues: one run on the batch under a GradientMode
        (RESET_AND_STEP by default); returns the objective (this rank's mean)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        exe, xbuf, tbuf, seed, loss, grads = self.training_state(x.shape[0])
        xbuf.upload(x)
        tbuf.upload(np.ascontiguousarray(target, dtype=np.int32 if self._loss == "ce" else np.float32))
        exe.run([xbuf, tbuf, seed] + self.param_buffers, [loss] + grads)
        self._optimizer.run(gradient_mode, grads)
        return float(loss.download(np.float32, (1,))[0])

    def zero_grad(self) -> None:
        """TrainingSession.zeroGrad: drops the pending gradient sum."""
        self._optimizer.zero_grad()

    def state(self) -> dict:
        """TrainingSession.state(): detached canonical (big-endian) parameter, optimizer-slot and
        pending-gradient bytes per parameter plus the two progress counters."""
        entries = []
        for index, (buf, shape) in enumerate(zip(self.param_buffers, self.param_shapes)):
            nbytes = int(np.prod(shape)) * 4
            entry = {"shape": tuple(shape), "parameter": buf.download_canonical(nbytes, 4),
                     "momentum": self._optimizer.state_canonical(index, 0),
                     "accumulated": self._optimizer.state_canonical(index, 2)}
            if not isinstance(self._optimizer_config, Sgd):
                entry["second"] = self._optimizer.state_canonical(index, 1)
            entries.append(entry)
        return {"optimizer_steps": self._optimizer.steps(), "accumulated_gradient_runs": self._optimizer.accumulated_runs(),
                "parameters": entries}

    def restore(self, state: dict) -> None:
        """TrainingSession.restore: the inverse of state()."""
        for index, (buf, entry) in enumerate(zip(self.param_buffers, state["parameters"])):
            buf.upload_canonical(entry["parameter"], 4)
            self._optimizer.restore_canonical(index, 0, entry["momentum"])
            if "second" in entry:
                self._optimizer.restore_canonical(index, 1, entry["second"])
            self._optimizer.restore_canonical(index, 2, entry["accumulated"])
        self._optimizer.set_progress(state["optimizer_steps"], state["accumulated_gradient_runs"])

    def gradients(self, x: np.ndarray, target: np.ndarray):
        """Runs forward and backward without stepping; returns (loss, [dW0, db0, ...])."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        exe, xbuf, tbuf, seed, loss, grads = self.training_state(x.shape[0])
        xbuf.upload(x)
        tbuf.upload(np.ascontiguousarray(target, dtype=np.int32 if self._loss == "ce" else np.float32))
        exe.run([xbuf, tbuf, seed] + self.param_buffers, [loss] + grads)
        return float(loss.download(np.float32, (1,))[0]), [g.download(np.float32, s) for g, s in zip(grads, self.param_shapes)]

    def optimizer_steps(self) -> int:
        return self._optimizer.steps() if self._optimizer else 0

    def optimizer_state(self, parameter_index: int, slot: int) -> np.ndarray:
        return self._optimizer.state(parameter_index, slot).reshape(self.param_shapes[parameter_index])

    def close(self) -> None:
        for exe, *_ in list(self._inference.values()) + list(self._training.values()):
            exe.close()
        if self._optimizer:
            self._optimizer.close()
