"""Library composition: one call wires the toolkit's services into a dependency container and runs extensions.

The reference composes its object graph in ``fairseq2/composition/lib.py:119-260`` (``_register_library``) and lets
third-party packages add to it through the ``fairseq2.extension`` entry-point group
(``fairseq2/composition/extensions.py:17-46``). Here the model / dataset / tokenizer families live in plain module
registries that recipes use directly; ``compose_library`` mirrors them, together with the process-wide services, into a
``DependencyContainer`` so that code written against a resolver (and extensions) sees one consistent view.
"""

from fairseq2_b200.composition.extensions import EXTENSION_GROUP as EXTENSION_GROUP
from fairseq2_b200.composition.extensions import ExtensionError as ExtensionError
from fairseq2_b200.composition.extensions import run_extensions as run_extensions
from fairseq2_b200.composition.library import compose_library as compose_library
from fairseq2_b200.composition.library import register_dataset_family as register_dataset_family
from fairseq2_b200.composition.library import register_model_family as register_model_family
from fairseq2_b200.composition.library import register_tokenizer_family as register_tokenizer_family
from fairseq2_b200.composition.library import register_checkpoint_models as register_checkpoint_models
from fairseq2_b200.composition.library import register_file_assets as register_file_assets
from fairseq2_b200.composition.library import register_in_memory_assets as register_in_memory_assets
from fairseq2_b200.composition.library import register_package_assets as register_package_assets
