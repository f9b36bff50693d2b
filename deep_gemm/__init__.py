"""Drop-in name: `import deep_gemm` resolves to the B200 implementation in `deepgemm_amd_b200`."""
from deepgemm_amd_b200 import *  # noqa: F401,F403
from deepgemm_amd_b200 import epilogue, testing, utils, __version__  # noqa: F401
