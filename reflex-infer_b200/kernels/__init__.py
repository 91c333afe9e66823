"""B200-native kernels behind reflex-infer's Python surface (paged-KV attention path).

Import names follow the reference's package (``README.md:117-125``):

    from kernels.kv_cache import kv_paged_append, kv_paged_lookup, kv_paged_scatter
    from kernels.rope import apply_rope, apply_rope_, build_rope_tables
    from kernels.softmax import online_softmax
    from kernels.attention import fused_attention

plus the fused paged entry points in ``kernels.attention`` (``paged_decode``,
``paged_attention``, ``rope_append``, ``paged_decode_step``, ``PagedWorkspace``).
Every function calls ``libreflex_b200.so`` through ``kernels._native``; there is no
Triton, no backend dispatch and no CPU path.
"""

__version__ = "0.1.0"
