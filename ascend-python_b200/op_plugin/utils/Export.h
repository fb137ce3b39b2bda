// Symbol visibility of the operator library (cf. op_plugin/utils/Export.h:24 of the reference).
#ifndef OP_PLUGIN_UTILS_EXPORT_H_
#define OP_PLUGIN_UTILS_EXPORT_H_

#if defined(__GNUC__)
#define OP_PLUGIN_HIDDEN __attribute__((visibility("hidden")))
#define OP_PLUGIN_EXPORT __attribute__((visibility("default")))
#else
#define OP_PLUGIN_HIDDEN
#define OP_PLUGIN_EXPORT
#endif

#endif  // OP_PLUGIN_UTILS_EXPORT_H_
