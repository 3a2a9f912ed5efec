"""GPT-2-small on the gradtuity_b200 modules: the training workload of the GEMM path."""
from .model import GPT2_SMALL, GPT2Block, GPT2Small  # noqa: F401
