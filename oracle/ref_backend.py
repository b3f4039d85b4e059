"""TEST INFRASTRUCTURE ONLY.  Adapters that let neoml_b200.resnet50.forward() run on the checkers:
RefBackend drives the reference's own CPU math engine (oracle/_ref), OracleBackend the plain-C oracle.
Both take and return numpy arrays in the channels-last blob layout."""
from __future__ import annotations

import numpy as np

from oracle_lib import Oracle, Reference


class _NumpyBackend:
    def __init__(self, impl):
        self.impl = impl
        self.conv_seconds = 0.0

    def upload(self, weights):
        return weights

    def conv(self, t, w, b, stride, pad, relu, residual):
        y = self.impl.blob_convolution(t, w, b, padding=(pad, pad), stride=(stride, stride))
        self.conv_seconds += getattr(self.impl, "last_seconds", 0.0)
        if residual is not None:
            y = self.add(y, residual)
        return self.relu(y) if relu else y

    def add(self, a, b):
        return self.impl.vector_op(3, a.ravel(), b.ravel()).reshape(a.shape)

    def relu(self, a):
        return self.impl.vector_op(9, a.ravel(), None, 0.0).reshape(a.shape)

    def max_pool_3x3_s2_p1(self, t):
        padded = self.impl.blob_resize_image(t, 1, 1, 1, 1, 0, 0.0)
        return self.impl.blob_max_pooling(padded, (3, 3), (2, 2))[0]

    def global_mean(self, t):
        n, h, w, c = t.shape
        s = self.impl.sum_matrix_rows(n, t.ravel(), h * w, c)
        return self.impl.vector_op(6, s.ravel(), None, 1.0 / (h * w)).reshape(n, c)

    def fully_connected(self, x, w, b):
        y = self.impl.multiply_matrix_by_transposed_matrix(x if hasattr(x, "data_ptr") else np.ascontiguousarray(x), w)
        return self.impl.add_vector_to_matrix_rows(1, y.ravel(), y.shape[0], y.shape[1], b).reshape(y.shape)

    def softmax(self, x):
        return self.impl.matrix_softmax_by_rows(x.ravel(), x.shape[0], x.shape[1]).reshape(x.shape)

    def argmax(self, x):
        return self.impl.find_max_value_in_rows(x.ravel(), x.shape[0], x.shape[1])[1]


class RefBackend(_NumpyBackend):
    def __init__(self):
        super().__init__(Reference())

    def close(self):
        self.impl.close()


class OracleBackend(_NumpyBackend):
    def __init__(self):
        super().__init__(Oracle())


class ShimmedEngineBackend(_NumpyBackend):
    """The B200 IMathEngine (C++ object, real virtual calls through the shim) behind the same graph; arrays are torch
    CUDA tensors.  The unfused call sequence only: that is what a CDnn issues."""

    def __init__(self, precision_flags: int = 0):
        from oracle_lib import ShimmedB200Engine
        super().__init__(ShimmedB200Engine(flags=precision_flags))

    def upload(self, weights):
        import torch
        return {k: torch.from_numpy(np.ascontiguousarray(v)).cuda() for k, v in weights.items()}

    def close(self):
        self.impl.close()
