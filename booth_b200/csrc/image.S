/* image.S -- embeds the sm_100a kernel image (a cubin built by nvcc from
 * the kernels directory) into libbooth_sm100.so, so the library needs no file at run time.
 * BOOTH_SM100_IMAGE is the path of the cubin, given by the build. */
    .section .rodata
    .balign 64
    .global booth_sm100_image
    .type booth_sm100_image, @object
booth_sm100_image:
    .incbin BOOTH_SM100_IMAGE
    .global booth_sm100_image_end
    .type booth_sm100_image_end, @object
booth_sm100_image_end:
    .byte 0
    .size booth_sm100_image, booth_sm100_image_end - booth_sm100_image
    .section .note.GNU-stack,"",@progbits
