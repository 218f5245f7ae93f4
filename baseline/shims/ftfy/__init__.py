"""Minimal stand-in for the third-party ``ftfy`` package, which is not installed in this image.

The reference's tokenizer module imports ``ftfy.fix_text`` at module scope; the parity tests import the
reference's text encoder (which imports that module) but never tokenize through it, so an identity function
is enough.  Nothing in ``solarwm_b200`` imports it."""
__version__ = "0.0.0+stub"


def fix_text(text, **_):
    return text
