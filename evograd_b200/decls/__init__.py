"""External evograd declarations; importable only where ``evograd`` is installed."""
