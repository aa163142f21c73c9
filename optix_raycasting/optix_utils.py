"""Same module path as the reference's OptiX host glue.  Only the constant that
other reference modules read from it (scripts/train.py:296) exists here; contexts,
pipelines and acceleration structures have no counterpart."""
from raygaussx_b200.render_optix import SIGMA_THRESHOLD  # noqa: F401
