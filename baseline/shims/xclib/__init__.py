"""Stand-in for pyxclib (not installable offline): the three entry points the reference imports."""
