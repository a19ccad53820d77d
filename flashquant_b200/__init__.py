"""B200 (sm_100a) kernels for the TurboQuant KV-cache hot path, behind the reference's names.

Importing the package does not load the native library; the first kernel call does, and it
raises if ``libflashquant_b200.so`` has not been built (``python -m flashquant_b200.build``).
"""

from .kernels import (  # noqa: F401
    HostDecodeStep,
    fused_tq_attention,
    fused_tq_attention_kv,
    pack_2bit,
    paged_decode_partials,
    paged_tq4_prefill,
    split_k_merge,
    split_k_paged_decode,
    split_k_paged_decode_multi,
    split_k_paged_decode_qjl,
    tq4_compress,
    tq4_compress_append,
    tq4_compress_append_qjl,
    tq4_compress_into,
    tq4_decompress,
    tq4_decompress_original,
    tq_prod_quantize,
    unpack_2bit,
)
from .cache import (  # noqa: F401
    CompressedBuffer,
    CompressedDynamicCache,
    FlashQuantCacheError,
    ValueCompressor,
)
from .quantizer import TurboQuantMSE, TurboQuantProd, haar_orthogonal, lloyd_max_codebook  # noqa: F401

__version__ = "0.1.0"
