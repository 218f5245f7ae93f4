"""Minimal stand-in for the third-party ``diffusers`` package, which is not installed in this image.

Only the three names the reference's Wan model imports are provided (``ConfigMixin``,
``register_to_config``, ``ModelMixin``); they carry no model, kernel or engine code.  The
stand-in is used by the reference arm of bench.py alone, so that the UNMODIFIED reference
classes under ``baseline/_ref`` can be constructed; nothing in ``solarwm_b200`` imports it."""
__version__ = "0.0.0+stub"
