"""Backend plugins (one package per model family); loaded lazily through the registry."""
