/* A caller-supplied xerbla_/cblas_xerbla, as the Netlib testers link in
 * (test/F77/dblat3.f:2768-2809, test/C/c_xerbla.c of the reference): records the
 * routine name and the argument index instead of printing.  Loaded with RTLD_GLOBAL
 * before the library, it must take precedence over the library's weak default. */
#include <string.h>
#include <stdarg.h>

int  hook_info = 0;
int  hook_calls = 0;
char hook_name[32] = "";

void xerbla_(const char rout[6], const int *info)
{
    hook_info = *info;
    hook_calls++;
    memcpy(hook_name, rout, 6);
    hook_name[6] = 0;
}

void cblas_xerbla(int info, const char *rout, const char *form, ...)
{
    (void)form;
    hook_info = info;
    hook_calls++;
    strncpy(hook_name, rout, sizeof hook_name - 1);
}
