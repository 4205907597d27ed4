"""fairseq2_b200: a B200-native (sm_100a) sequence-modeling toolkit.

``init_fairseq2_b200()`` composes the library once per process (cf. ``init_fairseq2`` in the reference's
``fairseq2/__init__.py``): it fills a ``DependencyContainer`` with the process-wide services and the model, dataset
and tokenizer families, runs the extensions published under the ``fairseq2_b200.extension`` entry-point group, and
installs the container as the process-global resolver. Importing the package does none of this; recipes and
``load_model`` work without it, the call is for code that resolves services from a container and for extensions.
"""

from __future__ import annotations

import threading
from typing import TYPE_CHECKING, Callable

__version__ = "0.1.0"

if TYPE_CHECKING:
    from fairseq2_b200.runtime.dependency import DependencyContainer

_lock = threading.Lock()
_container: "DependencyContainer | None" = None


def init_fairseq2_b200(*, extras: "Callable[[DependencyContainer], None] | None" = None,
                       no_extensions: bool = False) -> "DependencyContainer":
    """Composes the library (idempotent) and returns the container. ``extras`` runs after the built-in
    registrations and before the extensions, as in the reference."""
    global _container
    from fairseq2_b200.composition import compose_library, run_extensions
    from fairseq2_b200.runtime.dependency import DependencyContainer, set_dependency_resolver

    with _lock:
        if _container is not None:
            return _container
        container = DependencyContainer()
        compose_library(container)
        if extras is not None:
            extras(container)
        if not no_extensions:
            run_extensions(container)
        set_dependency_resolver(container)
        _container = container
        return container
