"""B200 (sm_100a) decode attention: MHA / GQA / MQA / MLA, one query token per sequence.

``decoding_attention_b200.interface`` holds the reference-compatible Python API (needs the built
torch extension), ``decoding_attention_b200.cabi`` the ctypes view of the C ABI,
``decoding_attention_b200.synth`` seeded synthetic workloads and ``decoding_attention_b200.sharded``
the multi-GPU partitioning helpers.  Nothing here computes attention on the CPU.
"""
__version__ = "0.1.0"


def __getattr__(name):
    if name in ("decoding_attn_fwd", "dmha_fwd", "dmla_fwd", "paged_fwd", "merge_partials"):
        from . import interface
        return getattr(interface, name)
    raise AttributeError(name)
