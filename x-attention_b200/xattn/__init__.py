"""Import-path compatibility with the reference project: `from xattn.src.Xattention import ...`."""
