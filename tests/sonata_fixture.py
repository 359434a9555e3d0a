"""The SONATA project writer lives in the package (bmtk_b200/sonata_writer.py); tests import it here."""
from bmtk_b200.sonata_writer import write_project  # noqa: F401
