"""B200-native masked flash-attention path of TAGSeq2TAGSeq (doc_causal / cross_doc_link), behind a C ABI.

Public surface:
    mask_spec   MaskSpec, mask creators with the reference's names, build_block_map (integer pre-pass)
    attention   masked_attn (torch operator with autograd), masked_attn_decode (one new token against cached K / V),
                flex_attention (drop-in signature)
    synth       seeded synthetic packs for benchmarks and tests
"""
from .mask_spec import (BlockMap, CrossDocLinkMaskCreator, DocSpan, LinkInfo, MaskSpec, build_block_map,  # noqa: F401
                        create_doc_causal_block_mask, from_reference, get_mask_creator, list_mask_creators,
                        make_mask_creator_callable, make_mask_creator_callable_from, read_status)


def __getattr__(name):  # attention registers torch custom ops; import it lazily
    if name in ("masked_attn", "masked_attn_decode", "flex_attention"):
        from . import attention
        return getattr(attention, name)
    raise AttributeError(name)
