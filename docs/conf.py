"""Sphinx configuration of the jigsaw_b200 documentation (``make -C docs html``).

Markdown pages are read through ``myst_parser``; the API reference (``api.rst``) is generated
from the docstrings by autosummary, one page per module of the package.
"""

from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.abspath(".."))

project = "jigsaw_b200"
author = "jigsaw_b200 developers"
release = "0.1"

extensions = [
    "sphinx.ext.autodoc",
    "sphinx.ext.autosummary",
    "sphinx.ext.napoleon",
    "sphinx.ext.viewcode",
    "myst_parser",
]
source_suffix = {".rst": "restructuredtext", ".md": "markdown"}
exclude_patterns = ["_build"]
master_doc = "index"

autosummary_generate = True
autosummary_imported_members = False
autodoc_default_options = {"members": True, "show-inheritance": True, "member-order": "bysource"}
autodoc_typehints = "description"
# the kernel library is loaded lazily, so importing the package for autodoc needs no GPU
autodoc_mock_imports: list[str] = []
napoleon_google_docstring = True
napoleon_numpy_docstring = False

html_theme = "sphinx_rtd_theme" if os.environ.get("JIGSAW_DOCS_THEME", "rtd") == "rtd" else "alabaster"
html_static_path: list[str] = []
myst_heading_anchors = 3
