"""Helpers shared by the GPU tests: seeded layers on the device in slot layout."""
import numpy as np
import torch

from oracle import deltazip_oracle as O


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


class DeviceLayer:
    """Base weight + `n_deltas` converted deltas, plus their oracle-side copies."""

    def __init__(self, n, k, n_deltas, bits, seed=0, num_slots=None):
        from deltazip_b200 import ops
        self.n, self.k, self.bits = n, k, bits
        self.w_np, self.deltas_np = O.make_layer(n, k, n_deltas, bits, seed=seed)
        self.num_slots = num_slots or max(n_deltas, 1)
        self.w = dev(self.w_np)
        self.qweight, self.meta, self.scales = ops.alloc_slots(self.num_slots, n, k, bits, "cuda")
        for d, (qw, qz, sc, _) in enumerate(self.deltas_np):
            ops.convert_from_gptq(dev(qw), dev(qz), dev(sc), bits,
                                  out=(self.qweight[d], self.meta[d], self.scales[d]))
        self._dense = None

    def oracle(self, x_np, idx_np):
        return O.apply_delta(x_np, self.w_np, self.deltas_np, idx_np)

    def dense(self):
        if self._dense is None:
            self._dense = [O.unpack(qw, qz, sc, b) for (qw, qz, sc, b) in self.deltas_np]
        return self._dense

    def oracle_fp32(self, x_np, idx_np):
        return O.apply_delta_dense(x_np, self.w_np, self.dense(), idx_np)
