"""Parts a decoder is put together from.  Importing the package registers the built-in
kinds (gqa_attention, swiglu, rmsnorm, rope); further kinds register themselves with the
decorators of `parts.base`."""
from . import base, spec  # noqa: F401
from . import attention, ffn, norm, rope  # noqa: F401  (register the built-in parts)
