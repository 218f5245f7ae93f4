"""Runtime services shared by all backends: rank algebra, fail-together error exchange, RNG
domains, create-only filesystem primitives, output layout and launch provenance."""
