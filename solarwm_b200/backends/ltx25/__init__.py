"""LTX backend (family ``ltx25_video``)."""


def create_backend(family: str):
    from .backend import LTX25Backend

    return LTX25Backend(family)
