"""Drop-in import name of the reference package (decoding_attn/__init__.py:15-19): call sites that
do ``from decoding_attn import decoding_attn_fwd`` keep working on top of the B200 library."""
from decoding_attention_b200 import __version__  # noqa: F401
from decoding_attention_b200.interface import decoding_attn_fwd, dmha_fwd, dmla_fwd, paged_fwd  # noqa: F401
