"""deltazip_b200: B200-native selective batched matmul for delta-compressed model serving.

Public surface mirrors the reference's delta-linear plugin
(serving/vllm/delta/): `apply_delta`, the `*WithDelta` layers, `DeltaConfig`,
`DeltaMapping`, `DeltaModelManager`.  The compute lives in
libdeltazip_b200.so (C ABI, include/deltazip_b200.h).
"""
from ._lib import DeltaZipError, lib  # noqa: F401

__version__ = "0.1.0"
