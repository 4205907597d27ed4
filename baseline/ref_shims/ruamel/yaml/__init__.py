"""Stand-in exposing the small part of ruamel.yaml's API that the reference
touches, implemented over PyYAML."""
import yaml as _yaml


class YAMLError(Exception):
    pass


class YAML:
    def __init__(self, typ="safe", pure=False):  # noqa: ARG002
        self.default_flow_style = False
        self.sort_base_mapping_type_on_output = False

    def load(self, stream):
        try:
            return _yaml.safe_load(stream)
        except _yaml.YAMLError as ex:  # pragma: no cover
            raise YAMLError(str(ex)) from ex

    def load_all(self, stream):
        try:
            yield from _yaml.safe_load_all(stream)
        except _yaml.YAMLError as ex:  # pragma: no cover
            raise YAMLError(str(ex)) from ex

    def dump(self, data, stream=None):
        return _yaml.safe_dump(data, stream, default_flow_style=False, sort_keys=False)

    def dump_all(self, docs, stream=None):
        return _yaml.safe_dump_all(docs, stream, default_flow_style=False, sort_keys=False)
