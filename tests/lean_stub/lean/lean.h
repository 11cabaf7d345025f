/* Stand-in for the Lean 4 runtime header: only the declarations lean/lean_ffi.cpp uses, with
 * the signatures of lean.h (Lean 4.28), so that the shim can be type-checked where no Lean
 * toolchain is installed.  Nothing here is implemented; never link against it. */
#pragma once
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
typedef struct lean_object lean_object;
typedef lean_object *lean_obj_arg;
typedef lean_object *b_lean_obj_arg;
typedef lean_object *lean_obj_res;
lean_obj_res lean_box(size_t n);
lean_obj_res lean_box_usize(size_t v);
lean_obj_res lean_box_uint32(uint32_t v);
size_t lean_unbox_usize(b_lean_obj_arg o);
lean_obj_res lean_io_result_mk_ok(lean_obj_arg a);
lean_obj_res lean_io_result_mk_error(lean_obj_arg e);
lean_obj_res lean_mk_io_user_error(lean_obj_arg str);
lean_obj_res lean_mk_string(const char *s);
size_t lean_array_size(b_lean_obj_arg o);
lean_object *lean_array_get_core(b_lean_obj_arg o, size_t i);
size_t lean_sarray_size(b_lean_obj_arg o);
uint8_t *lean_sarray_cptr(lean_object *o);
lean_obj_res lean_alloc_sarray(unsigned elem_size, size_t size, size_t capacity);
void lean_dec_ref(lean_object *o);
#ifdef __cplusplus
}
#endif
