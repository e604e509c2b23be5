"""Error types of the configuration layer."""


class ConfigError(ValueError):
    """A config.json that cannot be turned into a typed configuration: a missing
    required key, a value of the wrong type, or sizes that do not fit together."""


class UnknownArchitectureError(KeyError):
    """config.json names an architecture that nothing has registered."""

    def __str__(self) -> str:  # KeyError would print repr(args[0])
        return str(self.args[0]) if self.args else ""
