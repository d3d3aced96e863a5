"""rustinfer_b200: a small, whole inference engine for the Llama-3 dense decoder on one
B200 (sm_100a), with the capabilities RustInfer's decoder path shows."""
from .models import llama as _llama  # noqa: F401  (registers the architecture)

__version__ = "0.1.0"
