"""Versioned run configuration: strict loader, overrides, digests and the route table."""
from .loader import ResolvedConfig, canonical_json, load_config  # noqa: F401
from .routes import Route, resolve_route, supported_routes, validate_route  # noqa: F401
