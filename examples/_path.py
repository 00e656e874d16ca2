"""Puts the repository root on ``sys.path`` so that ``python examples/<name>.py`` works from a source checkout."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
