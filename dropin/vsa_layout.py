"""Re-export so that ``from vsa_layout import ...`` resolves to the B200 planner."""
from cudnn_vsa_b200.vsa_layout import BLOCK, SampleBlocks, Segment, VSALayout, build_vsa_layout  # noqa: F401
