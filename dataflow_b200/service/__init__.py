"""Engine service ("dataflowd"): server, wire protocol, client, store, resolver registry."""
from .client import EngineClient
from .registry import JitterResolver, list_resolvers, lookup_resolver, register_program_resolver
from .server import EngineConfig, Server
from .wire import ERROR_CODES, SCHEMA_VERSION, ServiceError, program_content_id
