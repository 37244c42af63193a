"""cake-b200: sm_100a backend for tpu-cake's matmul + reduce-scatter and ragged paged attention.

The directory name contains a hyphen, so the package is imported under the module name
``tpu_cake_b200`` through ``__graft_entry__.load_package()`` (tests, bench and the smoke entry all
use it). Importing the package does not load the CUDA library; the first plan built does, and
fails loudly when it is missing.
"""

__all__ = [
    "identity",
    "workloads",
    "cuda_lowering",
    "rpa_cuda_lowering",
    "mesh",
]
