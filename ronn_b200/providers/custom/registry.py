"""Registry of custom-hardware providers and their plugins
(crates/ronn-providers/src/custom/registry.rs:18-410).

A plugin is a Python module that exports ``ronn_plugin() -> ProviderPlugin``; ``discover_plugins`` scans the plugin
directories for ``*.py`` files (an optional ``<name>.plugin.json`` beside a file overrides the metadata the module
reports), checks ABI and minimum-version compatibility and keeps the metadata; ``load_plugin_from_file`` also creates
and registers the plugin's provider.  Registration, lookup, statistics and shutdown mirror the reference.
"""
from __future__ import annotations

import importlib.util
import json
import os
import threading
from dataclasses import dataclass
from typing import Dict, List, Optional

from ... import __version__ as RONN_VERSION
from ...api.errors import ProviderError
from .interface import (ABI_VERSION, CustomHardwareProvider, HardwareDevice, HardwareDiscovery, PluginMetadata,
                        ProviderPlugin)


def _version_tuple(v: str):
    out = []
    for part in v.split("."):
        digits = "".join(ch for ch in part if ch.isdigit())
        out.append(int(digits) if digits else 0)
    return tuple(out + [0] * (3 - len(out)))


@dataclass
class CustomRegistryStatistics:
    total_providers: int
    active_providers: int
    total_plugins: int
    loaded_plugins: int
    failed_plugins: int
    plugin_paths: List[str]


class DefaultHardwareDiscovery(HardwareDiscovery):
    """Finds nothing: a box without vendor plugins has no custom hardware."""

    def discover_devices(self) -> List[HardwareDevice]:
        return []


class CustomProviderRegistry:
    def __init__(self, plugin_paths: Optional[List[str]] = None, discovery: Optional[HardwareDiscovery] = None):
        self._lock = threading.RLock()
        self._providers: Dict[str, CustomHardwareProvider] = {}
        self._metadata: Dict[str, PluginMetadata] = {}
        self._paths: List[str] = list(plugin_paths or [])
        env = os.environ.get("RONN_PLUGIN_PATH")
        if env:
            self._paths += [p for p in env.split(os.pathsep) if p]
        self._discovery: HardwareDiscovery = discovery or DefaultHardwareDiscovery()

    # ------------------------------------------------------------------ plugins
    def add_plugin_path(self, path: str) -> None:
        with self._lock:
            if path not in self._paths:
                self._paths.append(str(path))

    def set_hardware_discovery(self, discovery: HardwareDiscovery) -> None:
        self._discovery = discovery

    def _load_module(self, path: str):
        name = "ronn_plugin_" + os.path.splitext(os.path.basename(path))[0]
        spec = importlib.util.spec_from_file_location(name, path)
        if spec is None or spec.loader is None:
            raise ProviderError(f"cannot import plugin '{path}'")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        factory = getattr(mod, "ronn_plugin", None)
        if factory is None:
            raise ProviderError(f"plugin '{path}' exports no ronn_plugin()")
        plugin = factory()
        if not isinstance(plugin, ProviderPlugin):
            raise ProviderError(f"plugin '{path}': ronn_plugin() must return a ProviderPlugin")
        return plugin

    def validate_plugin(self, md: PluginMetadata) -> None:
        if md.abi_version != ABI_VERSION:
            raise ProviderError(f"plugin '{md.name}' has ABI version {md.abi_version}, this runtime speaks {ABI_VERSION}")
        if _version_tuple(md.min_ronn_version) > _version_tuple(RONN_VERSION):
            raise ProviderError(f"plugin '{md.name}' needs runtime version {md.min_ronn_version} or newer "
                                f"(this is {RONN_VERSION})")
        if not md.name:
            raise ProviderError("plugin metadata carries no name")

    def _metadata_of(self, path: str, plugin: ProviderPlugin) -> PluginMetadata:
        md = plugin.get_metadata()
        md.plugin_path = path
        md.abi_version = plugin.get_abi_version()
        side = os.path.splitext(path)[0] + ".plugin.json"
        if os.path.isfile(side):
            with open(side) as f:
                for k, v in json.load(f).items():
                    if hasattr(md, k) and k not in ("plugin_path", "status"):
                        setattr(md, k, v)
        return md

    def discover_plugins(self) -> List[PluginMetadata]:
        """Imports every ``*.py`` of the plugin directories, records its metadata and status; loads no provider."""
        found = []
        with self._lock:
            for d in self._paths:
                if not os.path.isdir(d):
                    continue
                for fn in sorted(os.listdir(d)):
                    if not fn.endswith(".py") or fn.startswith("_"):
                        continue
                    path = os.path.join(d, fn)
                    try:
                        plugin = self._load_module(path)
                        md = self._metadata_of(path, plugin)
                        try:
                            self.validate_plugin(md)
                            md.status = "loaded" if plugin.is_hardware_available() else "disabled"
                        except ProviderError:
                            md.status = "incompatible"
                    except Exception as e:
                        md = PluginMetadata(os.path.splitext(fn)[0], plugin_path=path, status=f"load_error:{e}")
                    self._metadata[md.name] = md
                    found.append(md)
        return found

    def load_plugin_from_file(self, path: str, config: Optional[dict] = None) -> str:
        """Imports a plugin module, validates it, creates its provider and registers it; returns the provider name."""
        plugin = self._load_module(path)
        md = self._metadata_of(path, plugin)
        self.validate_plugin(md)
        if not plugin.is_hardware_available():
            md.status = "disabled"
            with self._lock:
                self._metadata[md.name] = md
            raise ProviderError(f"plugin '{md.name}': its hardware is not available on this machine")
        provider = plugin.create_provider(config)
        self.register_provider(provider.provider_name(), provider, md)
        return provider.provider_name()

    # ------------------------------------------------------------------ providers
    def register_provider(self, name: str, provider: CustomHardwareProvider, metadata: Optional[PluginMetadata] = None) -> None:
        with self._lock:
            if name in self._providers:
                raise ProviderError(f"Provider '{name}' is already registered")
            if not provider.is_hardware_available():
                raise ProviderError(f"Hardware not available for provider '{name}'")
            provider.initialize()
            self._providers[name] = provider
            if metadata is not None:
                metadata.status = "loaded"
                self._metadata[metadata.name] = metadata

    def get_provider(self, name: str) -> Optional[CustomHardwareProvider]:
        with self._lock:
            return self._providers.get(name)

    def list_providers(self) -> List[str]:
        with self._lock:
            return sorted(self._providers)

    def get_plugin_metadata(self, name: str) -> Optional[PluginMetadata]:
        return self._metadata.get(name)

    def get_all_plugin_metadata(self) -> Dict[str, PluginMetadata]:
        return dict(self._metadata)

    def unregister_provider(self, name: str) -> None:
        with self._lock:
            p = self._providers.pop(name, None)
            if p is None:
                raise ProviderError(f"Provider '{name}' is not registered")
            p.shutdown()

    def discover_hardware(self) -> List[HardwareDevice]:
        return self._discovery.discover_devices()

    def as_execution_provider(self, name: str, options=None):
        """The registered provider wrapped for ``Model.create_session`` (``ProviderType.CUSTOM``)."""
        from .interface import CustomProviderAdapter
        p = self.get_provider(name)
        if p is None:
            raise ProviderError(f"Provider '{name}' is not registered")
        return CustomProviderAdapter(p, options)

    def get_statistics(self) -> CustomRegistryStatistics:
        with self._lock:
            loaded = sum(1 for m in self._metadata.values() if m.status == "loaded")
            failed = sum(1 for m in self._metadata.values() if m.status.startswith("load_error") or m.status == "incompatible")
            active = sum(1 for p in self._providers.values() if p.is_hardware_available())
            return CustomRegistryStatistics(len(self._providers), active, len(self._metadata), loaded, failed, list(self._paths))

    def shutdown(self) -> None:
        with self._lock:
            errors = []
            for name, p in list(self._providers.items()):
                try:
                    p.shutdown()
                except Exception as e:                 # keep going: every provider gets its shutdown call
                    errors.append(f"{name}: {e}")
            self._providers.clear()
            if errors:
                raise ProviderError("errors while shutting providers down: " + "; ".join(errors))
