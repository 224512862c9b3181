"""Re-export so that ``from vsa import ...`` resolves to the B200 implementation."""
from cudnn_vsa_b200.vsa import *  # noqa: F401,F403
from cudnn_vsa_b200.vsa import block_wo_padding_to_raster, raster_to_block_wo_padding, vsa_attention  # noqa: F401
