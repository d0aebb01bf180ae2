"""The benchmark configurations (topologies, seeded weight files, seeded inputs) live in the package, where the
benchmark uses them too; the tests reach them under the old name."""
from spingalett_b200.configs import *  # noqa: F401,F403
