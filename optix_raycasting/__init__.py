"""Import-path shim: lets the reference's callers keep their own import lines,
``from optix_raycasting import render_optix as r_ox`` (scripts/train.py:13) and
``from optix_raycasting import optix_utils as u_ox``, while getting the B200
implementation.  Nothing OptiX-related lives here."""
