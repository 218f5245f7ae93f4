import functools
import inspect


class _Config(dict):
    def __getattr__(self, name):
        try:
            return self[name]
        except KeyError as exc:
            raise AttributeError(name) from exc


class ConfigMixin:
    config_name = "config.json"
    ignore_for_config = []

    def register_to_config(self, **kwargs):
        if not hasattr(self, "_internal_dict"):
            self._internal_dict = _Config()
        self._internal_dict.update(kwargs)

    @property
    def config(self):
        return self._internal_dict

    @classmethod
    def from_config(cls, config, **kwargs):
        if not isinstance(config, dict):
            import json
            from pathlib import Path

            config = json.loads(Path(config).read_text())
        accepted = set(inspect.signature(cls.__init__).parameters)
        args = {k: v for k, v in {**config, **kwargs}.items() if k in accepted and not k.startswith("_")}
        return cls(**args)


def register_to_config(init):
    @functools.wraps(init)
    def inner(self, *args, **kwargs):
        sig = inspect.signature(init)
        bound = sig.bind(self, *args, **kwargs)
        bound.apply_defaults()
        values = {k: v for k, v in bound.arguments.items() if k != "self" and k not in getattr(self, "ignore_for_config", [])}
        init(self, *args, **kwargs)
        self.register_to_config(**values)

    return inner
