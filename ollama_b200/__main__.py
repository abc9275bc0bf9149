"""``python -m ollama_b200 ...`` runs the command line."""
import sys

from .cli.main import main

sys.exit(main())
