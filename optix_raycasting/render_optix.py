"""Same module path as the reference's autograd entry point; re-exports the B200 implementation."""
from raygaussx_b200.render_optix import (RenderOptixFunction, RenderOptixSettings, Renderer, get_renderer,  # noqa: F401
                                         render_full, SIGMA_THRESHOLD, TRANSMITTANCE_EPSILON)
