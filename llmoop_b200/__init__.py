"""llmoop_b200: B200 (sm_100a) backend for the MTP speculative decode path of
compiled NERVE packages.  The product is the C-ABI library libnerve_b200.so
(include/nerve_b200.h); this package is its thin Python mirror, the package
tooling (synthetic checkpoints, native package writer) and the build step.
There is no CPU fallback: every compute call needs the CUDA library and a GPU.
"""

from .runtime import (  # noqa: F401
    Engine,
    NerveError,
    Package,
    RunReport,
    library,
    nccl_library_path,
    tensor_parallel_unique_id,
    tp_shard_range,
    validate_package,
    verify_prefix,
)
