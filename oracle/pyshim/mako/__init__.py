"""Stand-in for the `mako` package (not installed here), written for this
repository's tests: only `mako.template.Template` with plain ${name}
substitution. Templates that use mako control lines ("% for", "% if") are
refused, which is how pygpu.reduction's own code generator announces itself
as unavailable in this environment."""
