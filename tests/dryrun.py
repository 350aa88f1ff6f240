"""The compile-only backend lives in the package (neon_b200/dryrun.py); tests import it from here."""
from neon_b200.dryrun import DryRunBackend, DryTensor          # noqa: F401
