"""Test helpers: the seeded generators live in straydog_b200.synthetic."""
from straydog_b200.synthetic import *  # noqa: F401,F403
