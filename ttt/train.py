"""``python -m ttt.train`` == ``python -m dttt_b200.train``."""
import sys

from dttt_b200.train import *  # noqa: F401,F403
from dttt_b200.train import main

if __name__ == "__main__":
    sys.exit(main())
