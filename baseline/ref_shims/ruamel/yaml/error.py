from ruamel.yaml import YAMLError  # noqa: F401
