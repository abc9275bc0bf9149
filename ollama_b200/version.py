"""Version string reported by ``/api/version`` and the CLI."""
VERSION = "0.1.0-b200"
