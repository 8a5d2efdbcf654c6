"""``python -m bloomery_b200.serve``: the server binary (``bloomery_serve.rs`` in the reference)."""
import sys

from .cli import main

sys.exit(main())
