"""MiniMax-H3 backend (family ``minimax_h3``)."""


def create_backend(family: str):
    from .backend import MiniMaxH3Backend

    return MiniMaxH3Backend(family)
