"""e3nn-style ``o3`` namespace (``src/o3/__init__.py`` in the reference): irreps and spherical harmonics."""

from .irreps import Irrep, Irreps


def __getattr__(name):
    if name == "SphericalHarmonics":
        from .modules import SphericalHarmonics

        return SphericalHarmonics
    if name == "spherical_harmonics":
        from .spherical_harmonics import spherical_harmonics

        return spherical_harmonics
    raise AttributeError(f"{__name__} has no attribute {name!r}")


__all__ = ["Irrep", "Irreps", "SphericalHarmonics", "spherical_harmonics"]
