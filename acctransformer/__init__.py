"""The reference's import surface, served by the B200 library.

``pip install`` of the reference puts a package called ``acctransformer`` on the path
(train/setup.py:22-31) and its users import through it
(train/acctransformer/flash_attention/nn/layer/flash_attention.py:27).  The modules below
carry the same names at the same paths and re-export the ``acctransformer_b200`` classes and
functions, so that

    from acctransformer.flash_attention.nn.layer.flash_attention import FlashAttention
    from acctransformer.triangle_attention.triangle_attention import TriangleAttention
    from acctransformer.flash_attention.ops.flash_attention.flash_attention_impl import get_flash_attention

resolve unchanged.  Nothing else lives here.
"""
