"""Wan2.2 backend (families ``wan22_ti2v_5b`` and ``wan22_i2v_a14b``)."""


def create_backend(family: str):
    from .backend import Wan22Backend

    return Wan22Backend(family)
