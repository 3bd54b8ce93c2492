"""The error every configuration reader raises, whatever the architecture."""


class ConfigError(ValueError):
    """A config.json (or an engine option) that cannot be run; the message names the key."""
