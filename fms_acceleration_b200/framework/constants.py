"""Names shared by the framework core.  Same values as fms_acceleration/constants.py:15-24 of the reference."""

# root key of the acceleration configuration YAML
KEY_PLUGINS = "plugins"
# plugin packages are discovered under this module-name prefix
PLUGIN_PREFIX = "fms_acceleration_"
# environment variable that may carry the path of the configuration file
ACCELERATION_FRAMEWORK_ENV_KEY = "ACCELERATION_FRAMEWORK_CONFIG_FILE"
# import order == registration order == activation precedence (the two model loaders come first)
PLUGINS = ["peft", "foak", "aadp", "moe", "odm", "mcp"]
