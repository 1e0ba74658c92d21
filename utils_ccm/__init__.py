"""Import-compatibility package: scripts written against the reference import its helper modules
as `utils_ccm.<module>`; each name here re-exports the implementation in fastcache_b200."""
