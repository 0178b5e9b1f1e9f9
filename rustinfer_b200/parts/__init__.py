"""Parts a decoder is put together from.  Importing the package registers the built-in
kinds (gqa_attention, gated_linear_attention, delta_rule, parallel_mixers, swiglu, dense_mlp,
rmsnorm, layernorm, rope); further kinds register themselves with the
decorators of `parts.base`."""
from . import base, spec  # noqa: F401
from . import attention, ffn, linear_attention, norm, parallel, rope, stem_tail  # noqa: F401  (register the built-in parts)
