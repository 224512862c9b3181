"""Re-export so that ``from vsa_kernels import ...`` resolves to the B200 row kernels."""
from cudnn_vsa_b200.vsa_kernels import (  # noqa: F401
    BLOCK, block_w_padding_to_block_wo_padding, block_w_padding_to_raster,
    block_wo_padding_to_block_w_padding, gather, raster_to_block_w_padding, reorder_tokens)
