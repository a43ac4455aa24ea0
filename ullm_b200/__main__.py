"""`python -m ullm_b200 ...` is the offline command line of `ullm_b200.engine.cli`."""

import sys

from .engine.cli import main

sys.exit(main())
