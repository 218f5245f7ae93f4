"""Expected-failure hierarchy.  The CLI maps these (plus OSError / ValueError) to exit code 2
(reference: solar/errors.py:4-21, solar/cli.py:430-446)."""


class SolarWMError(RuntimeError):
    """Base of every failure the framework raises on purpose."""


class ConfigurationError(SolarWMError):
    """The resolved run configuration breaks a public contract."""


class DataContractError(SolarWMError):
    """An index row, sample, camera or tensor breaks the data contract."""


class BackendContractError(SolarWMError):
    """A backend cannot serve the requested route."""


class CheckpointError(SolarWMError):
    """A checkpoint transaction or a resume-compatibility gate failed."""
